"""apply_transform_config (transform/apply.py:26 of the reference)."""
import torch

from .factory.base import TransformFactory
from .transform_config import TransformConfig

__all__ = ["apply_transform_config"]


def apply_transform_config(model: torch.nn.Module, config: TransformConfig, seed=None) -> None:
    for name, scheme in config.config_groups.items():
        TransformFactory.from_scheme(scheme, name=name, seed=seed).apply_to_model(model)
    model.transform_config = config
