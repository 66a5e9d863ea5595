"""MXFP4 scale helpers on the GPU, with the reference's names and argument meaning
(quantization/utils/mxfp4_utils.py:25 convert_mxfp4_exp_scale, :43 round_to_power_2,
:75 generate_mxfp4_scales).  Scales are powers of two stored as uint8 exponents."""
import torch

from ... import torch_ops as ops

__all__ = ["convert_mxfp4_exp_scale", "generate_mxfp4_scales", "round_to_power_2"]


def convert_mxfp4_exp_scale(scale: torch.Tensor, dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """uint8 exponent scale -> 2 ** (scale - 127) in `dtype`."""
    assert scale.dtype == torch.uint8
    return ops.mxfp4_convert_scales(scale, dtype)


def round_to_power_2(x: torch.Tensor) -> torch.Tensor:
    """Round bf16 values to the closest power of two (sign and exponent kept, mantissa dropped after adding a
    quarter of its range)."""
    assert x.dtype == torch.bfloat16
    return ops.mxfp4_round_pow2(x)


def generate_mxfp4_scales(x: torch.Tensor) -> torch.Tensor:
    """bf16 block maxima -> uint8 exponents: round to a power of two, take its exponent, subtract the e2m1
    exponent range (2), bias by 127, clamp to uint8."""
    assert x.dtype == torch.bfloat16
    return ops.mxfp4_generate_scales(x)
