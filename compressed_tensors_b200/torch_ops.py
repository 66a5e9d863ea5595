"""The codec kernels as torch custom operators: ``torch.ops.ctb200.<name>``.

Each operator wraps one C-ABI entry point (through compressed_tensors_b200.ops, which allocates the outputs and
passes raw pointers and the current stream) and carries a fake implementation that returns the right shapes and
dtypes without touching data, so that meta / fake tensors, ``torch.compile`` and ``torch.export`` see through the
calls.  The functions of this module have the signatures of their namesakes in ``ops`` and dispatch through the
operators; the host mirror of the reference interface calls these.

Operators: quantize, dequantize, fake_quantize, absmax_quantize, minmax, calculate_qparams, generate_gparam,
pack_int32, unpack_int32, pack_fp4, unpack_fp4, pack_bitmasks, unpack_bitmasks, sparse24_mask, sparse24_compress,
quantize_fp8_sparse24, sparse24_decompress, sparse24_decompress_dequantize_fp8, bitmask_compress, bitmask_decompress, hadamard.
"""
from typing import List, Optional, Sequence, Tuple

import torch
from torch import Tensor
from torch.library import custom_op

from . import ops as _o
from .ops import *  # noqa: F401,F403  (everything without an operator of its own is used as it is)
from .ops import QFLOAT, QINT, ROT_TENSOR, _packed_shape

NS = "ctb200"


def _prec_str(precision) -> str:
    return "tensor" if precision == ROT_TENSOR else str(precision).replace("torch.", "")


def _prec_val(precision: str):
    return ROT_TENSOR if precision == "tensor" else getattr(torch, precision)


# ---------------------------------------------------------------- quantize / dequantize / fake_quantize

@custom_op(f"{NS}::quantize", mutates_args=())
def _quantize(x: Tensor, scale: Tensor, zp: Optional[Tensor], qtype: int, bits: int, col_group: int, row_group: int,
              scale_row_stride: int, out_dtype: Optional[torch.dtype], codec: str, g_idx: Optional[Tensor],
              global_scale: Optional[Tensor]) -> Tensor:
    return _o.quantize(x, scale, zp, qtype=qtype, bits=bits, col_group=col_group, row_group=row_group,
                       scale_row_stride=scale_row_stride, out_dtype=out_dtype, codec=codec, g_idx=g_idx, global_scale=global_scale)


@_quantize.register_fake
def _(x, scale, zp, qtype, bits, col_group, row_group, scale_row_stride, out_dtype, codec, g_idx, global_scale):
    if codec == "pack32":
        return x.new_empty(_packed_shape(x.shape, x.shape[-1], codec, bits), dtype=torch.int32)
    if codec == "fp4x2":
        return x.new_empty(_packed_shape(x.shape, x.shape[-1], codec, bits), dtype=torch.uint8)
    return x.new_empty(x.shape, dtype=out_dtype)


def quantize(x, scale, zp=None, *, qtype, bits, col_group, row_group=1, scale_row_stride, out_dtype=None, codec="dtype",
             g_idx=None, global_scale=None):
    return torch.ops.ctb200.quantize(x, scale, zp, qtype, bits, col_group, row_group, scale_row_stride, out_dtype, codec, g_idx, global_scale)


@custom_op(f"{NS}::dequantize", mutates_args=())
def _dequantize(q: Tensor, scale: Tensor, zp: Optional[Tensor], qtype: int, bits: int, col_group: int, row_group: int,
                scale_row_stride: int, out_dtype: torch.dtype, codec: str, cols: Optional[int], g_idx: Optional[Tensor],
                global_scale: Optional[Tensor]) -> Tensor:
    return _o.dequantize(q, scale, zp, qtype=qtype, bits=bits, col_group=col_group, row_group=row_group,
                         scale_row_stride=scale_row_stride, out_dtype=out_dtype, codec=codec, cols=cols, g_idx=g_idx,
                         global_scale=global_scale)


@_dequantize.register_fake
def _(q, scale, zp, qtype, bits, col_group, row_group, scale_row_stride, out_dtype, codec, cols, g_idx, global_scale):
    if codec == "dtype":
        cols = q.shape[-1]
    elif codec == "fp4x2":
        cols = q.shape[-1] * 2
    elif cols is None:
        raise ValueError("cols is required for packed input")
    return q.new_empty(tuple(q.shape[:-1]) + (cols,), dtype=out_dtype)


def dequantize(q, scale, zp=None, *, qtype, bits, col_group, row_group=1, scale_row_stride, out_dtype, codec="dtype", cols=None,
               g_idx=None, global_scale=None):
    return torch.ops.ctb200.dequantize(q, scale, zp, qtype, bits, col_group, row_group, scale_row_stride, out_dtype, codec,
                                       None if cols is None else int(cols), g_idx, global_scale)


@custom_op(f"{NS}::fake_quantize", mutates_args=())
def _fake_quantize(x: Tensor, scale: Tensor, zp: Optional[Tensor], qtype: int, bits: int, col_group: int, row_group: int,
                   scale_row_stride: int, out_dtype: torch.dtype, g_idx: Optional[Tensor], global_scale: Optional[Tensor]) -> Tensor:
    return _o.fake_quantize(x, scale, zp, qtype=qtype, bits=bits, col_group=col_group, row_group=row_group,
                            scale_row_stride=scale_row_stride, out_dtype=out_dtype, g_idx=g_idx, global_scale=global_scale)


@_fake_quantize.register_fake
def _(x, scale, zp, qtype, bits, col_group, row_group, scale_row_stride, out_dtype, g_idx, global_scale):
    return x.new_empty(x.shape, dtype=out_dtype)


def fake_quantize(x, scale, zp=None, *, qtype, bits, col_group, row_group=1, scale_row_stride, out_dtype, g_idx=None, global_scale=None):
    return torch.ops.ctb200.fake_quantize(x, scale, zp, qtype, bits, col_group, row_group, scale_row_stride, out_dtype, g_idx, global_scale)


@custom_op(f"{NS}::absmax_quantize", mutates_args=())
def _absmax_quantize(x: Tensor, qtype: int, bits: int, col_group: int, codec: str, out_dtype: Optional[torch.dtype],
                     global_scale: Optional[Tensor], hadamard_n: int, signs: Optional[Tensor], precision: str) -> Tuple[Tensor, Tensor]:
    return _o.absmax_quantize(x, qtype=qtype, bits=bits, col_group=col_group, codec=codec, out_dtype=out_dtype,
                              global_scale=global_scale, hadamard_n=hadamard_n, signs=signs, precision=_prec_val(precision))


@_absmax_quantize.register_fake
def _(x, qtype, bits, col_group, codec, out_dtype, global_scale, hadamard_n, signs, precision):
    cols = x.shape[-1]
    sdt = torch.float8_e4m3fn if (qtype == QFLOAT and bits == 4) else x.dtype
    scale = x.new_empty(tuple(x.shape[:-1]) + (cols // col_group,), dtype=sdt)
    if codec == "pack32":
        out = x.new_empty(_packed_shape(x.shape, cols, codec, bits), dtype=torch.int32)
    elif codec == "fp4x2":
        out = x.new_empty(_packed_shape(x.shape, cols, codec, bits), dtype=torch.uint8)
    else:
        out = x.new_empty(x.shape, dtype=out_dtype)
    return out, scale


def absmax_quantize(x, *, qtype, bits, col_group, codec="pack32", out_dtype=None, global_scale=None, hadamard_n=0, signs=None,
                    precision=torch.float64):
    return torch.ops.ctb200.absmax_quantize(x, qtype, bits, col_group, codec, out_dtype, global_scale, hadamard_n, signs, _prec_str(precision))


# ---------------------------------------------------------------- quantization parameters

@custom_op(f"{NS}::minmax", mutates_args=())
def _minmax(x: Tensor, row_group: int, col_group: int) -> Tuple[Tensor, Tensor]:
    return _o.minmax(x, row_group, col_group)


@_minmax.register_fake
def _(x, row_group, col_group):
    cols = x.shape[-1]
    rows = x.numel() // cols
    shape = (rows // row_group, cols // col_group)
    return x.new_empty(shape), x.new_empty(shape)


def minmax(x, row_group, col_group):
    return torch.ops.ctb200.minmax(x, int(row_group), int(col_group))


@custom_op(f"{NS}::calculate_qparams", mutates_args=())
def _calculate_qparams(mins: Tensor, maxs: Tensor, qtype: int, bits: int, symmetric: bool, global_scale: Optional[Tensor]) -> Tuple[Tensor, Tensor]:
    return _o.calculate_qparams(mins, maxs, qtype=qtype, bits=bits, symmetric=symmetric, global_scale=global_scale)


@_calculate_qparams.register_fake
def _(mins, maxs, qtype, bits, symmetric, global_scale):
    fp4 = qtype == QFLOAT and bits == 4
    sdt = torch.float8_e4m3fn if (fp4 and global_scale is not None) else mins.dtype
    return mins.new_empty(mins.shape, dtype=sdt), mins.new_empty(mins.shape, dtype=torch.int8 if qtype == QINT else torch.float8_e4m3fn)


def calculate_qparams(mins, maxs, *, qtype, bits, symmetric, global_scale=None):
    return torch.ops.ctb200.calculate_qparams(mins, maxs, qtype, bits, bool(symmetric), global_scale)


@custom_op(f"{NS}::generate_gparam", mutates_args=())
def _generate_gparam(mn: Tensor, mx: Tensor) -> Tensor:
    return _o.generate_gparam(mn, mx)


@_generate_gparam.register_fake
def _(mn, mx):
    return mn.new_empty(1, dtype=torch.float32)


def generate_gparam(mn, mx):
    return torch.ops.ctb200.generate_gparam(mn, mx)


# ---------------------------------------------------------------- stand-alone packing

@custom_op(f"{NS}::pack_int32", mutates_args=())
def _pack_int32(value: Tensor, bits: int, packed_dim: int) -> Tensor:
    return _o.pack_int32(value, bits, packed_dim)


@_pack_int32.register_fake
def _(value, bits, packed_dim):
    if value.dtype is not torch.int8:
        raise ValueError("Tensor must be quantized to torch.int8 before packing")
    if bits > 8:
        raise ValueError("Packing is only supported for less than 8 bits")
    pf = 32 // bits
    if packed_dim == 0:
        return value.new_empty((value.shape[1], (value.shape[0] + pf - 1) // pf), dtype=torch.int32).transpose(0, 1)
    return value.new_empty((value.shape[0], (value.shape[1] + pf - 1) // pf), dtype=torch.int32)


def pack_int32(value, bits, packed_dim=1):
    return torch.ops.ctb200.pack_int32(value, int(bits), int(packed_dim))


@custom_op(f"{NS}::unpack_int32", mutates_args=())
def _unpack_int32(words: Tensor, bits: int, shape: List[int], packed_dim: int) -> Tensor:
    return _o.unpack_int32(words, bits, shape, packed_dim)


@_unpack_int32.register_fake
def _(words, bits, shape, packed_dim):
    if words.dtype is not torch.int32:
        raise ValueError(f"Expected {torch.int32} but got {words.dtype}, Aborting unpack.")
    if packed_dim == 0:
        return words.new_empty((words.shape[1], int(shape[0])), dtype=torch.int8).transpose(0, 1)
    return words.new_empty((words.shape[0], int(shape[1])), dtype=torch.int8)


def unpack_int32(words, bits, shape, packed_dim=1):
    return torch.ops.ctb200.unpack_int32(words, int(bits), [int(s) for s in shape], int(packed_dim))


@custom_op(f"{NS}::pack_fp4", mutates_args=())
def _pack_fp4(x: Tensor) -> Tensor:
    return _o.pack_fp4(x)


@_pack_fp4.register_fake
def _(x):
    m, n = x.shape
    if n % 2 != 0:
        raise ValueError("tensor must have an even number of columns for nvfp4 compression")
    return x.new_empty((m, n // 2), dtype=torch.uint8)


def pack_fp4(x):
    return torch.ops.ctb200.pack_fp4(x)


@custom_op(f"{NS}::unpack_fp4", mutates_args=())
def _unpack_fp4(a: Tensor, m: int, n: int, dtype: torch.dtype) -> Tensor:
    return _o.unpack_fp4(a, m, n, dtype)


@_unpack_fp4.register_fake
def _(a, m, n, dtype):
    return a.new_empty((m, n), dtype=dtype)


def unpack_fp4(a, m, n, dtype=torch.bfloat16):
    return torch.ops.ctb200.unpack_fp4(a, int(m), int(n), dtype)


@custom_op(f"{NS}::pack_bitmasks", mutates_args=())
def _pack_bitmasks(bytemasks: Tensor) -> Tensor:
    return _o.pack_bitmasks(bytemasks)


@_pack_bitmasks.register_fake
def _(bytemasks):
    return bytemasks.new_empty(tuple(bytemasks.shape[:-1]) + ((bytemasks.shape[-1] + 7) // 8,), dtype=torch.uint8)


def pack_bitmasks(bytemasks):
    return torch.ops.ctb200.pack_bitmasks(bytemasks)


@custom_op(f"{NS}::unpack_bitmasks", mutates_args=())
def _unpack_bitmasks(packed: Tensor, shape: List[int]) -> Tensor:
    return _o.unpack_bitmasks(packed, shape)


@_unpack_bitmasks.register_fake
def _(packed, shape):
    return packed.new_empty(tuple(int(s) for s in shape), dtype=torch.bool)


def unpack_bitmasks(packed, shape):
    return torch.ops.ctb200.unpack_bitmasks(packed, [int(s) for s in shape])


# ---------------------------------------------------------------- sparse codecs

@custom_op(f"{NS}::sparse24_mask", mutates_args=())
def _sparse24_mask(x: Tensor) -> Tensor:
    return _o.sparse24_mask(x)


@_sparse24_mask.register_fake
def _(x):
    if x.numel() % 4 != 0:
        raise ValueError("Tensor size must be a multiple of 4 for TWO_FOUR sparsity")
    return x.new_empty(x.shape, dtype=torch.bool)


def sparse24_mask(x):
    return torch.ops.ctb200.sparse24_mask(x)


@custom_op(f"{NS}::sparse24_compress", mutates_args=())
def _sparse24_compress(x: Tensor) -> Tuple[Tensor, Tensor]:
    return _o.sparse24_compress(x)


@_sparse24_compress.register_fake
def _(x):
    rows, cols = x.shape
    if x.numel() % 4 != 0:
        raise ValueError("Tensor size must be a multiple of 4 for TWO_FOUR sparsity")
    return x.new_empty((rows, cols // 2)), x.new_empty((rows, (cols + 7) // 8), dtype=torch.uint8)


def sparse24_compress(x):
    return torch.ops.ctb200.sparse24_compress(x)


@custom_op(f"{NS}::quantize_fp8_sparse24", mutates_args=())
def _quantize_fp8_sparse24(x: Tensor, scale: Tensor, zero_point: Optional[Tensor] = None) -> Tuple[Tensor, Tensor]:
    return _o.quantize_fp8_sparse24(x, scale, zero_point)


@_quantize_fp8_sparse24.register_fake
def _(x, scale, zero_point=None):
    rows, cols = x.shape
    if cols % 8 != 0:
        raise ValueError("fused FP8 + 2:4 compression needs cols % 8 == 0")
    return x.new_empty((rows, cols // 2), dtype=torch.float8_e4m3fn), x.new_empty((rows, cols // 8), dtype=torch.uint8)


def quantize_fp8_sparse24(x, scale, zero_point=None):
    return torch.ops.ctb200.quantize_fp8_sparse24(x, scale, zero_point)


@custom_op(f"{NS}::sparse24_decompress", mutates_args=())
def _sparse24_decompress(values: Tensor, bitmask: Tensor, shape: List[int]) -> Tensor:
    return _o.sparse24_decompress(values, bitmask, shape)


@_sparse24_decompress.register_fake
def _(values, bitmask, shape):
    return bitmask.new_empty((int(shape[0]), int(shape[1])), dtype=values.dtype)


def sparse24_decompress(values, bitmask, shape):
    return torch.ops.ctb200.sparse24_decompress(values, bitmask, [int(s) for s in shape])


@custom_op(f"{NS}::sparse24_decompress_dequantize_fp8", mutates_args=())
def _sparse24_decompress_dequantize_fp8(values: Tensor, bitmask: Tensor, scale: Tensor, shape: List[int]) -> Tensor:
    return _o.sparse24_decompress_dequantize_fp8(values, bitmask, scale, shape)


@_sparse24_decompress_dequantize_fp8.register_fake
def _(values, bitmask, scale, shape):
    return bitmask.new_empty((int(shape[0]), int(shape[1])), dtype=torch.bfloat16)


def sparse24_decompress_dequantize_fp8(values, bitmask, scale, shape):
    return torch.ops.ctb200.sparse24_decompress_dequantize_fp8(values, bitmask, scale, [int(s) for s in shape])


@custom_op(f"{NS}::bitmask_compress", mutates_args=())
def _bitmask_compress(x: Tensor) -> Tuple[Tensor, Tensor, Tensor]:
    values, bitmask, row_offsets = _o.bitmask_compress(x)
    return values.clone(), bitmask, row_offsets  # `values` is a slice of a full-capacity buffer: hand out its own storage


@_bitmask_compress.register_fake
def _(x):
    rows, cols = x.shape
    nnz = torch.library.get_ctx().new_dynamic_size()  # as many values as the tensor has non-zeros: known only from the data
    return x.new_empty((nnz,)), x.new_empty((rows, (cols + 7) // 8), dtype=torch.uint8), x.new_empty((rows,), dtype=torch.int64)


def bitmask_compress(x):
    return torch.ops.ctb200.bitmask_compress(x)


@custom_op(f"{NS}::bitmask_decompress", mutates_args=())
def _bitmask_decompress(values: Tensor, bitmask: Tensor, shape: List[int]) -> Tensor:
    return _o.bitmask_decompress(values, bitmask, shape)


@_bitmask_decompress.register_fake
def _(values, bitmask, shape):
    return bitmask.new_empty((int(shape[0]), int(shape[1])), dtype=values.dtype)


def bitmask_decompress(values, bitmask, shape):
    return torch.ops.ctb200.bitmask_decompress(values, bitmask, [int(s) for s in shape])


# ---------------------------------------------------------------- Hadamard rotation

@custom_op(f"{NS}::hadamard", mutates_args=())
def _hadamard(x: Tensor, n: int, signs: Optional[Tensor], inverse: bool, side: int, precision: str, normalize: bool) -> Tensor:
    return _o.hadamard(x, n, signs=signs, inverse=inverse, side=side, precision=_prec_val(precision), normalize=normalize)


@_hadamard.register_fake
def _(x, n, signs, inverse, side, precision, normalize):
    return x.new_empty(x.shape)


def hadamard(x, n, signs=None, inverse=False, side=0, precision=torch.float64, normalize=True):
    return torch.ops.ctb200.hadamard(x, int(n), signs, bool(inverse), int(side), _prec_str(precision), bool(normalize))


OPERATORS: Sequence[str] = ("quantize", "dequantize", "fake_quantize", "absmax_quantize", "minmax", "calculate_qparams",
                            "generate_gparam", "pack_int32", "unpack_int32", "pack_fp4", "unpack_fp4", "pack_bitmasks",
                            "unpack_bitmasks", "sparse24_mask", "sparse24_compress", "quantize_fp8_sparse24", "sparse24_decompress", "sparse24_decompress_dequantize_fp8",
                            "bitmask_compress", "bitmask_decompress", "hadamard")
