"""`naive-quantized` / `int-quantized` / `float-quantized`: one int8 or e4m3 element per weight
(compressors/quantized_compressors/naive_quantized.py of the reference)."""
from typing import Dict, Optional, Tuple

import torch
from torch import Tensor

from ...config import CompressionFormat
from ...quantization.lifecycle.forward import dequantize, quantize
from ...quantization.quant_args import QuantizationArgs
from ..base import BaseCompressor
from .base import BaseQuantizationCompressor

__all__ = ["NaiveQuantizationCompressor", "IntQuantizationCompressor", "FloatQuantizationCompressor"]

_FLOATS = (torch.bfloat16, torch.float16, torch.float32)


@BaseCompressor.register(name=CompressionFormat.naive_quantized.value)
class NaiveQuantizationCompressor(BaseQuantizationCompressor):
    @property
    def compression_param_names(self) -> Tuple[str]:
        return ("weight", "weight_scale", "weight_zero_point", "weight_g_idx")

    def compression_param_info(self, weight_shape: torch.Size, quantization_args: Optional[QuantizationArgs] = None):
        return {"weight": (weight_shape, quantization_args.pytorch_dtype())}

    def compress_weight(self, weight: Tensor, scale: Tensor, quantization_args: QuantizationArgs, zero_point: Optional[Tensor] = None,
                        g_idx: Optional[Tensor] = None, device: Optional[torch.device] = None,
                        global_scale: Optional[Tensor] = None) -> Dict[str, Tensor]:
        if global_scale is not None:
            raise ValueError("global_scale is not supported for the NaiveQuantizationCompressor")
        if weight.dtype in _FLOATS:
            q = quantize(x=weight, scale=scale, zero_point=zero_point, g_idx=g_idx, args=quantization_args,
                         dtype=quantization_args.pytorch_dtype())
        else:
            q = weight
        if device is not None:
            q = q.to(device)
        return {"weight": q}

    def decompress_weight(self, compressed_data: Dict[str, Tensor], quantization_args: Optional[QuantizationArgs] = None) -> Tensor:
        w = compressed_data["weight"]
        return dequantize(x_q=w, scale=compressed_data["weight_scale"].to(w.device),
                          zero_point=None if compressed_data.get("weight_zero_point") is None else compressed_data["weight_zero_point"].to(w.device),
                          g_idx=compressed_data.get("weight_g_idx"))


@BaseCompressor.register(name=CompressionFormat.int_quantized.value)
class IntQuantizationCompressor(NaiveQuantizationCompressor):
    pass


@BaseCompressor.register(name=CompressionFormat.float_quantized.value)
class FloatQuantizationCompressor(NaiveQuantizationCompressor):
    pass
