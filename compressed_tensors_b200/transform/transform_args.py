"""TransformArgs / TransformLocation (transform/transform_args.py of the reference)."""
from enum import Enum
from typing import List

from pydantic import BaseModel, ConfigDict, Field, field_validator

__all__ = ["TransformArgs", "TransformLocation"]


class TransformLocation(str, Enum):
    INPUT = "input"
    WEIGHT_INPUT = "weight_input"
    WEIGHT_OUTPUT = "weight_output"
    OUTPUT = "output"
    K_CACHE = "k_cache"
    Q_ATTN = "q_attn"

    def is_online(self) -> bool:
        return self not in (TransformLocation.WEIGHT_INPUT, TransformLocation.WEIGHT_OUTPUT)


class TransformArgs(BaseModel, use_enum_values=True):
    targets: List[str]
    location: TransformLocation
    inverse: bool = Field(default=False)
    ignore: List[str] = Field(default_factory=list)

    model_config = ConfigDict(extra="forbid")

    @field_validator("targets", "ignore", mode="before")
    def _wrap(cls, value):
        return [value] if isinstance(value, str) else value

    def is_online(self) -> bool:
        return TransformLocation(self.location).is_online()
