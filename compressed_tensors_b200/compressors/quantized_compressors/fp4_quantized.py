"""`nvfp4-pack-quantized`: e2m1 codes two per byte with e4m3 group scales and an fp32 global scale
(compressors/quantized_compressors/fp4_quantized.py of the reference).  compress_weight and
decompress_weight are one fused kernel each."""
from typing import Dict, Optional, Tuple

import torch
from torch import Tensor

from ... import torch_ops as ops
from ...config import CompressionFormat
from ...quantization.lifecycle.forward import _geometry
from ...quantization.quant_args import QuantizationArgs
from ..base import BaseCompressor
from .base import BaseQuantizationCompressor

__all__ = ["pack_fp4_to_uint8", "unpack_fp4_from_uint8", "NVFP4PackedCompressor", "MXFP4PackedCompressor"]


def pack_fp4_to_uint8(x: torch.Tensor) -> torch.Tensor:
    """fp4_quantized.py:135-178: values on the e2m1 grid -> uint8 [m, n/2]; the even column goes in
    the low nibble, bit 3 of a nibble is the sign bit of the value (so -0.0 packs as 0x8)."""
    m, n = x.shape
    if n % 2 != 0:
        raise ValueError("tensor must have an even number of columns for nvfp4 compression")
    return ops.pack_fp4(x)


def unpack_fp4_from_uint8(a: torch.Tensor, m: int, n: int, dtype: Optional[torch.dtype] = torch.bfloat16) -> torch.Tensor:
    """fp4_quantized.py:187-221."""
    assert a.dtype == torch.uint8
    return ops.unpack_fp4(a, m, n, dtype)


@BaseCompressor.register(name=CompressionFormat.nvfp4_pack_quantized.value)
class NVFP4PackedCompressor(BaseQuantizationCompressor):
    @property
    def compression_param_names(self) -> Tuple[str]:
        return ("weight_packed", "weight_scale", "weight_zero_point", "weight_global_scale")

    def compression_param_info(self, weight_shape: torch.Size, quantization_args: Optional[QuantizationArgs] = None):
        return {"weight_packed": (torch.Size((weight_shape[0], weight_shape[1] // 2)), torch.uint8)}

    def compress_weight(self, weight: Tensor, scale: Tensor, global_scale: Tensor, quantization_args: QuantizationArgs,
                        device: Optional[torch.device] = None, zero_point: Optional[Tensor] = None,
                        g_idx: Optional[Tensor] = None) -> Dict[str, Tensor]:
        if weight.shape[-1] % 2 != 0:
            raise ValueError("tensor must have an even number of columns for nvfp4 compression")
        cg, rg, srs = _geometry(weight, scale, quantization_args)
        packed = ops.quantize(weight, scale, zero_point, qtype=ops.QFLOAT, bits=4, col_group=cg, row_group=rg, scale_row_stride=srs,
                              codec="fp4x2", global_scale=global_scale)
        if device is not None:
            packed = packed.to(device)
        return {"weight_packed": packed}

    def decompress_weight(self, compressed_data: Dict[str, Tensor], quantization_args: Optional[QuantizationArgs] = None) -> Tensor:
        packed = compressed_data["weight_packed"]
        scale = compressed_data["weight_scale"].to(packed.device)
        gs = compressed_data["weight_global_scale"].to(packed.device)
        m, n2 = packed.shape
        groups = scale.shape[-1]
        return ops.dequantize(packed, scale, None, qtype=ops.QFLOAT, bits=4, col_group=(2 * n2) // groups, scale_row_stride=groups,
                              out_dtype=torch.bfloat16, codec="fp4x2", global_scale=gs)


@BaseCompressor.register(name=CompressionFormat.mxfp4_pack_quantized.value)
class MXFP4PackedCompressor(NVFP4PackedCompressor):
    pass
