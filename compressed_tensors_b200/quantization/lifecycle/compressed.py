"""compress_quantized_weights (quantization/lifecycle/compressed.py:31-76 of the reference): replace a module's
weight by its int8 codes, on the GPU."""
import torch
from torch.nn import Module

from ..quant_config import QuantizationStatus
from .forward import quantize

__all__ = ["compress_quantized_weights"]


def compress_quantized_weights(module: Module) -> None:
    """Apply to a whole model with `model.apply(compress_quantized_weights)`."""
    scheme = getattr(module, "quantization_scheme", None)
    if not scheme or not scheme.weights:
        return
    if getattr(module, "quantization_status", None) is QuantizationStatus.COMPRESSED:
        return
    weight, scale = getattr(module, "weight", None), getattr(module, "weight_scale", None)
    if weight is None or scale is None:
        module.quantization_status = QuantizationStatus.COMPRESSED  # consistent status throughout the model
        return
    module.weight.requires_grad = False
    module.weight.data = quantize(x=weight, scale=scale, zero_point=getattr(module, "weight_zero_point", None),
                                  g_idx=getattr(module, "weight_g_idx", None), args=scheme.weights, dtype=torch.int8)
    module.quantization_status = QuantizationStatus.COMPRESSED
