"""TransformScheme (transform/transform_scheme.py of the reference)."""
from typing import List, Optional

import torch
from pydantic import BaseModel, ConfigDict, Field, field_serializer, field_validator

from .transform_args import TransformArgs

__all__ = ["TransformScheme"]


class TransformScheme(BaseModel):
    type: str
    apply: List[TransformArgs] = Field(default_factory=list)
    randomize: bool = Field(default=False)
    requires_grad: bool = Field(default=False)
    head_dim: Optional[int] = Field(default=None)
    precision: torch.dtype = Field(default=torch.float32)

    model_config = ConfigDict(extra="forbid", arbitrary_types_allowed=True)

    @field_validator("precision", mode="before")
    def _precision(cls, value):
        if isinstance(value, str):
            return getattr(torch, value.replace("torch.", ""))
        return value

    @field_serializer("precision")
    def _ser_precision(self, value: torch.dtype):
        return str(value)
