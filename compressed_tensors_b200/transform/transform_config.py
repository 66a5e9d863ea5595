"""TransformConfig (transform/transform_config.py of the reference)."""
from typing import Dict

from pydantic import BaseModel, ConfigDict

from .transform_scheme import TransformScheme

__all__ = ["TransformConfig"]


class TransformConfig(BaseModel):
    config_groups: Dict[str, TransformScheme]

    model_config = ConfigDict(extra="forbid")
