"""`pack-quantized`: int4/int8 codes packed into int32 words
(compressors/quantized_compressors/pack_quantized.py of the reference).  compress_weight is ONE kernel
(quantize fused with the packing), decompress_weight is ONE kernel (unpacking fused with dequantize)."""
import math
from typing import Dict, Literal, Optional, Tuple, Union

import torch
from torch import Tensor

from ... import torch_ops as ops
from ...config import CompressionFormat
from ...quantization.lifecycle.forward import _geometry, dequantize, infer_dequant_args, quantize
from ...quantization.quant_args import QuantizationArgs, QuantizationStrategy
from ..base import BaseCompressor
from .base import BaseQuantizationCompressor

__all__ = ["PackedQuantizationCompressor", "pack_to_int32", "unpack_from_int32"]

_PACKED_ZP = (QuantizationStrategy.GROUP.value, QuantizationStrategy.CHANNEL.value)
_FLOATS = (torch.bfloat16, torch.float16, torch.float32)


def pack_to_int32(value: torch.Tensor, num_bits: int, packed_dim: Union[Literal[0], Literal[1]] = 1) -> torch.Tensor:
    """pack_quantized.py:186-246: int8 codes -> int32 words, element i of a run in bits
    [num_bits*i, num_bits*(i+1)) after adding 2^(num_bits-1); padding fields are zero.
    `packed_dim=0` packs down the rows and returns a transposed view, like the reference."""
    return ops.pack_int32(value, num_bits, packed_dim)


def unpack_from_int32(value: torch.Tensor, num_bits: int, shape: torch.Size,
                      packed_dim: Union[Literal[0], Literal[1]] = 1) -> torch.Tensor:
    """pack_quantized.py:249-309."""
    return ops.unpack_int32(value, num_bits, shape, packed_dim)


@BaseCompressor.register(name=CompressionFormat.pack_quantized.value)
class PackedQuantizationCompressor(BaseQuantizationCompressor):
    @property
    def compression_param_names(self) -> Tuple[str]:
        return ("weight_packed", "weight_scale", "weight_zero_point", "weight_g_idx", "weight_shape")

    def compression_param_info(self, weight_shape: torch.Size, quantization_args: Optional[QuantizationArgs] = None):
        pf = 32 // quantization_args.num_bits
        info = {
            "weight_packed": (torch.Size((weight_shape[0], math.ceil(weight_shape[1] / pf))), torch.int32),
            "weight_shape": (torch.Size((2,)), torch.int32),
        }
        if not quantization_args.symmetric and quantization_args.strategy in _PACKED_ZP:
            zp_factor = quantization_args.group_size if quantization_args.strategy == QuantizationStrategy.GROUP.value else weight_shape[-1]
            info["weight_zero_point"] = (torch.Size((math.ceil(weight_shape[0] / pf), weight_shape[-1] // zp_factor)), torch.int32)
        return info

    def compress_weight(self, weight: Tensor, scale: Tensor, quantization_args: QuantizationArgs, zero_point: Optional[Tensor] = None,
                        g_idx: Optional[Tensor] = None, device: Optional[torch.device] = None,
                        global_scale: Optional[Tensor] = None) -> Dict[str, Tensor]:
        if global_scale is not None:
            raise ValueError("global_scale is not supported for the PackQuantizationCompressor")
        bits = quantization_args.num_bits
        if weight.dtype in _FLOATS:
            if g_idx is not None and bool((g_idx == -1).any()):
                g_idx = None
            cg, rg, srs = _geometry(weight, scale, quantization_args)
            packed = ops.quantize(weight, scale, zero_point, qtype=ops.QINT, bits=bits, col_group=cg, row_group=rg,
                                  scale_row_stride=srs, codec="pack32", g_idx=g_idx)
        else:  # already quantized to int8
            packed = pack_to_int32(weight, bits)
        shape = torch.tensor(weight.shape)
        if device is not None:
            packed, shape = packed.to(device), shape.to(device)
        out = {"weight_shape": shape, "weight_packed": packed}
        if not quantization_args.symmetric and quantization_args.strategy in _PACKED_ZP:
            out["weight_zero_point"] = pack_to_int32(zero_point, bits, packed_dim=0).contiguous()
        return out

    def decompress_weight(self, compressed_data: Dict[str, Tensor], quantization_args: Optional[QuantizationArgs] = None) -> Tensor:
        words = compressed_data["weight_packed"]
        scale = compressed_data["weight_scale"]
        zero_point = compressed_data.get("weight_zero_point")
        g_idx = compressed_data.get("weight_g_idx")
        shape = torch.Size(int(s) for s in compressed_data["weight_shape"])
        bits = quantization_args.num_bits
        dev = words.device
        scale = scale.to(dev)
        if not quantization_args.symmetric and quantization_args.strategy in _PACKED_ZP:
            assert zero_point is not None, "Asymmetric quantization requires zero-point values"
            zero_point = unpack_from_int32(zero_point.to(dev), bits, (shape[0], scale.shape[-1]), packed_dim=0).contiguous()
        elif zero_point is not None:
            zero_point = zero_point.to(dev)
        if g_idx is not None and bool((g_idx == -1).any()):
            g_idx = None
        # the reference dequantizes with args=None: the strategy comes from the scale's shape
        probe = torch.empty(shape, dtype=torch.int8, device="meta")
        args = infer_dequant_args(probe, scale)
        cg, rg, srs = _geometry(probe, scale, args)
        grouped = args.strategy in (QuantizationStrategy.GROUP, QuantizationStrategy.TENSOR_GROUP)
        return ops.dequantize(words, scale, zero_point, qtype=ops.QINT, bits=bits, col_group=cg, row_group=rg, scale_row_stride=srs,
                              out_dtype=scale.dtype, codec="pack32", cols=shape[1],
                              g_idx=g_idx.to(dev) if (g_idx is not None and grouped) else None)
