"""Quantization-parameter helpers with the reference's signatures (quantization/utils/helpers.py),
computed on the device by the ctb200 kernels."""
import math
from typing import Optional, Tuple

import torch

from ... import torch_ops as ops
from ..quant_args import FP4_E2M1_DATA, FP8_E4M3_DATA, FloatArgs, QuantizationArgs, QuantizationStrategy, QuantizationType

__all__ = ["calculate_qparams", "compute_dynamic_scales_and_zp", "calculate_range", "generate_gparam", "is_fp4", "strategy_cdiv", "qtype_code"]


def is_fp4(quantization_args: QuantizationArgs) -> bool:
    return quantization_args.num_bits == 4 and quantization_args.type == QuantizationType.FLOAT


def qtype_code(args: QuantizationArgs) -> int:
    if args.type == QuantizationType.INT:
        return ops.QINT
    if args.type == QuantizationType.FLOAT:
        if args.num_bits not in (4, 8):
            raise NotImplementedError("Range calculation only supported for 4 and 8 bits")
        return ops.QFLOAT
    raise ValueError(f"Invalid quantization type {args.type}")


def calculate_range(quantization_args: QuantizationArgs, device) -> Tuple[torch.Tensor, torch.Tensor]:
    """helpers.py:208-234: (q_min, q_max) as 0-dim tensors."""
    if quantization_args.type == QuantizationType.INT:
        r = 2 ** quantization_args.num_bits
        lo, hi = -r / 2, r / 2 - 1
    elif quantization_args.type == QuantizationType.FLOAT:
        if quantization_args.num_bits == 8:
            lo, hi = FP8_E4M3_DATA.min, FP8_E4M3_DATA.max
        elif quantization_args.num_bits == 4:
            lo, hi = FP4_E2M1_DATA.min, FP4_E2M1_DATA.max
        else:
            raise NotImplementedError("Range calculation only supported for 4 and 8 bits")
    else:
        raise ValueError(f"Invalid quantization type {quantization_args.type}")
    return torch.tensor(lo, device=device), torch.tensor(hi, device=device)


def calculate_qparams(min_vals: torch.Tensor, max_vals: torch.Tensor, quantization_args: QuantizationArgs,
                      global_scale: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """helpers.py:67-146.  Scales come back in the dtype of min/max (e4m3 for fp4 with a global
    scale), zero points in the quantized dtype; 0-dim inputs give shape [1]."""
    qtype = qtype_code(quantization_args)
    if is_fp4(quantization_args) and not quantization_args.symmetric:
        raise NotImplementedError("Asymmetric Quantization is not supported for FP4")
    scale, zp = ops.calculate_qparams(min_vals, max_vals, qtype=qtype, bits=quantization_args.num_bits,
                                      symmetric=quantization_args.symmetric,
                                      global_scale=global_scale if is_fp4(quantization_args) else None)
    if scale.ndim == 0:
        scale, zp = scale.reshape(1), zp.reshape(1)
    return scale, zp


def compute_dynamic_scales_and_zp(value: torch.Tensor, args: QuantizationArgs, module=None,
                                  global_scale: Optional[torch.Tensor] = None):
    """helpers.py:149-205: min/max over the strategy's reduction dims, then calculate_qparams."""
    strategy = args.strategy
    cols = value.shape[-1]
    if strategy == QuantizationStrategy.TOKEN:
        if value.ndim <= 2:  # nothing left to reduce per token: the reference falls back to one scale
            mn, mx = ops.minmax(value, value.numel() // cols, cols)
            mn, mx = mn.reshape(()), mx.reshape(())
        else:
            inner = math.prod(value.shape[2:])
            mn, mx = ops.minmax(value.reshape(-1, inner), 1, inner)
            shape = tuple(value.shape[:2]) + (1,) * (value.ndim - 2)
            mn, mx = mn.reshape(shape), mx.reshape(shape)
    elif strategy == QuantizationStrategy.TENSOR:
        mn, mx = ops.minmax(value, value.numel() // cols, cols)
        mn, mx = mn.reshape(()), mx.reshape(())
    elif strategy in (QuantizationStrategy.TENSOR_GROUP, QuantizationStrategy.GROUP):
        g = args.group_size
        if cols % g != 0:
            raise ValueError(f"tensor column shape must be divisble by the given group_size {g} but got {cols}")
        mn, mx = ops.minmax(value, 1, g)
        shape = tuple(value.shape[:-1]) + (cols // g,)
        mn, mx = mn.reshape(shape), mx.reshape(shape)
    else:
        ok = (QuantizationStrategy.TOKEN, QuantizationStrategy.TENSOR, QuantizationStrategy.TENSOR_GROUP, QuantizationStrategy.GROUP)
        raise ValueError("Dynamic quantization is only supported for ", f"{ok}")
    return calculate_qparams(mn, mx, args, global_scale=global_scale)


def generate_gparam(updated_min_val: torch.Tensor, updated_max_val: torch.Tensor, scale_data: Optional[FloatArgs] = FP8_E4M3_DATA,
                    quant_data: Optional[FloatArgs] = FP4_E2M1_DATA, dtype: Optional[torch.dtype] = torch.float32) -> torch.Tensor:
    """helpers.py:414-434: 448 * 6 / amax in the dtype of the extrema, returned as `dtype` [1]."""
    if scale_data is not FP8_E4M3_DATA or quant_data is not FP4_E2M1_DATA:
        raise NotImplementedError("only the e4m3 scale / e2m1 value pairing is built")
    return ops.generate_gparam(updated_min_val, updated_max_val).to(dtype)


def strategy_cdiv(value: int, divisor: int, strategy: Optional[QuantizationStrategy], strict: bool = False) -> int:
    dividend = math.ceil(value / divisor)
    if dividend * divisor != value and strict:
        raise ValueError(f"{strategy} quantization strategy requires strict division of weight/activation size {value} "
                         f"and group/block size {divisor}.")
    return dividend
