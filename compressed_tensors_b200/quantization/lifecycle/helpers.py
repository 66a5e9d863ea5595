"""Switches for the wrapped quantized forward (quantization/lifecycle/helpers.py:28-33 of the reference)."""
from torch.nn import Module

__all__ = ["enable_quantization", "disable_quantization"]


def enable_quantization(module: Module) -> None:
    module.quantization_enabled = True


def disable_quantization(module: Module) -> None:
    module.quantization_enabled = False
