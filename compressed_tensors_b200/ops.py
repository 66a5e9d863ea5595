"""Tensor-level wrappers over the C ABI: allocate outputs with torch, pass raw pointers and the
current CUDA stream, turn status codes into exceptions.  Every function launches hand-written
sm_100a kernels; none has a CPU path."""
import ctypes
from typing import Optional, Tuple

import torch

from . import _lib as L
from ._lib import CODE_DTYPE, CODE_FP4X2, CODE_PACK32, DT, QFLOAT, QINT, QDesc, check, i32, i64, lib, ptr, require_cuda, stream_of

__all__ = [
    "quantize", "dequantize", "fake_quantize", "minmax", "calculate_qparams", "generate_gparam",
    "mxfp4_round_pow2", "mxfp4_generate_scales", "mxfp4_convert_scales",
    "cutlass24_compress", "cutlass24_decompress", "marlin24_pack_weight", "marlin24_pack_scales",
    "pack_int32", "unpack_int32", "pack_fp4", "unpack_fp4", "pack_bitmasks", "unpack_bitmasks",
    "sparse24_mask", "sparse24_compress", "quantize_fp8_sparse24", "sparse24_decompress", "sparse24_decompress_dequantize_fp8", "bitmask_compress", "bitmask_decompress", "hadamard",
    "absmax_quantize", "rotate_quantize_int4_batch", "rotate_quantize_int4_batch_bounded", "quantize_pack_int4_batch",
    "unpack_dequantize_int4_batch", "quantize_fp8_channel_batch", "dequantize_fp8_channel_batch",
    "quantize_fp4_g16_batch", "dequantize_fp4_g16_batch", "tensor_table", "QINT", "QFLOAT",
]

_CODEC = {"dtype": CODE_DTYPE, "pack32": CODE_PACK32, "fp4x2": CODE_FP4X2}
ROT_TENSOR = "tensor"  # value of `precision` that runs the block-128 rotation on the tensor cores (tcgen05)


def _precision_code(precision) -> int:
    return 100 if precision == ROT_TENSOR else DT[precision]


def _c(t: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
    return None if t is None else t.contiguous()


def _desc(rows, cols, col_group, row_group, srs, qtype, bits, x_dtype, scale, zp, q_dtype, codec) -> QDesc:
    return QDesc(rows, cols, col_group, row_group, srs, qtype, bits, DT[x_dtype], DT[scale.dtype],
                 DT[zp.dtype] if zp is not None else L.I8, DT[q_dtype] if q_dtype is not None else 0, _CODEC[codec], 0)


def _gs(global_scale, like):
    if global_scale is None:
        return None
    return global_scale.to(device=like.device, dtype=torch.float32).contiguous()


def _gidx(g_idx, like):
    return None if g_idx is None else g_idx.to(device=like.device, dtype=torch.int32).contiguous()


def _packed_shape(shape, cols, codec, bits):
    lead = tuple(shape[:-1])
    if codec == "pack32":
        pf = 32 // bits
        return lead + ((cols + pf - 1) // pf,)
    if codec == "fp4x2":
        return lead + (cols // 2,)
    return tuple(shape)


def quantize(x, scale, zp=None, *, qtype, bits, col_group, row_group=1, scale_row_stride, out_dtype=None,
             codec="dtype", g_idx=None, global_scale=None):
    """quantization/lifecycle/forward.py:45 quantize, optionally fused with pack_to_int32
    (codec="pack32") or pack_fp4_to_uint8 (codec="fp4x2")."""
    require_cuda(x, scale, zp)
    x, scale, zp = _c(x), _c(scale), _c(zp)
    cols = x.shape[-1]
    rows = x.numel() // cols if cols else 0
    if codec == "pack32":
        out = torch.empty(_packed_shape(x.shape, cols, codec, bits), dtype=torch.int32, device=x.device)
    elif codec == "fp4x2":
        out = torch.empty(_packed_shape(x.shape, cols, codec, bits), dtype=torch.uint8, device=x.device)
    else:
        out = torch.empty(x.shape, dtype=out_dtype, device=x.device)
    d = _desc(rows, cols, col_group, row_group, scale_row_stride, qtype, bits, x.dtype, scale, zp, out_dtype, codec)
    gs, gi = _gs(global_scale, x), _gidx(g_idx, x)
    check(lib().ctb_quantize(ctypes.byref(d), ptr(x), ptr(scale), ptr(zp), ptr(gi), ptr(gs), ptr(out), stream_of(x)))
    return out


def dequantize(q, scale, zp=None, *, qtype, bits, col_group, row_group=1, scale_row_stride, out_dtype,
               codec="dtype", cols=None, g_idx=None, global_scale=None):
    """forward.py:85 dequantize; `q` may be pack_to_int32 words (codec="pack32", pass the dense
    column count as `cols`) or pack_fp4_to_uint8 bytes (codec="fp4x2")."""
    require_cuda(q, scale, zp)
    q, scale, zp = _c(q), _c(scale), _c(zp)
    if codec == "dtype":
        cols = q.shape[-1]
    elif codec == "fp4x2":
        cols = q.shape[-1] * 2
    elif cols is None:
        raise ValueError("cols is required for packed input")
    rows = q.numel() // q.shape[-1] if q.shape[-1] else 0
    out = torch.empty(tuple(q.shape[:-1]) + (cols,), dtype=out_dtype, device=q.device)
    d = _desc(rows, cols, col_group, row_group, scale_row_stride, qtype, bits, out_dtype, scale, zp,
              q.dtype if codec == "dtype" else None, codec)
    gs, gi = _gs(global_scale, q), _gidx(g_idx, q)
    check(lib().ctb_dequantize(ctypes.byref(d), ptr(q), ptr(scale), ptr(zp), ptr(gi), ptr(gs), ptr(out), stream_of(q)))
    return out


def fake_quantize(x, scale, zp=None, *, qtype, bits, col_group, row_group=1, scale_row_stride, out_dtype,
                  g_idx=None, global_scale=None):
    """forward.py:157 fake_quantize."""
    require_cuda(x, scale, zp)
    x, scale, zp = _c(x), _c(scale), _c(zp)
    cols = x.shape[-1]
    rows = x.numel() // cols if cols else 0
    out = torch.empty(x.shape, dtype=out_dtype, device=x.device)
    d = _desc(rows, cols, col_group, row_group, scale_row_stride, qtype, bits, x.dtype, scale, zp, out_dtype, "dtype")
    gs, gi = _gs(global_scale, x), _gidx(g_idx, x)
    check(lib().ctb_fake_quantize(ctypes.byref(d), ptr(x), ptr(scale), ptr(zp), ptr(gi), ptr(gs), ptr(out), stream_of(x)))
    return out


def minmax(x, row_group, col_group) -> Tuple[torch.Tensor, torch.Tensor]:
    """amin / amax over [row_group x col_group] tiles of x viewed as [rows, cols]
    (quantization/utils/helpers.py:149-205)."""
    require_cuda(x)
    x = _c(x)
    cols = x.shape[-1]
    rows = x.numel() // cols
    shape = (rows // row_group, cols // col_group)
    mn = torch.empty(shape, dtype=x.dtype, device=x.device)
    mx = torch.empty(shape, dtype=x.dtype, device=x.device)
    nbytes = lib().ctb_minmax_workspace_bytes(rows, cols, row_group, col_group)
    ws = torch.empty(max(int(nbytes), 1), dtype=torch.uint8, device=x.device) if nbytes else None
    check(lib().ctb_minmax(ptr(x), i32(DT[x.dtype]), i64(rows), i64(cols), i64(row_group), i64(col_group),
                           ptr(mn), ptr(mx), ptr(ws), stream_of(x)))
    return mn, mx


def calculate_qparams(mins, maxs, *, qtype, bits, symmetric, global_scale=None):
    """helpers.py:67 calculate_qparams on device."""
    require_cuda(mins, maxs)
    mins, maxs = _c(mins), _c(maxs)
    fp4 = qtype == QFLOAT and bits == 4
    zp_dtype = torch.int8 if qtype == QINT else torch.float8_e4m3fn
    sdt = torch.float8_e4m3fn if (fp4 and global_scale is not None) else mins.dtype
    scale = torch.empty(mins.shape, dtype=sdt, device=mins.device)
    zp = torch.empty(mins.shape, dtype=zp_dtype, device=mins.device)
    gs = _gs(global_scale, mins)
    check(lib().ctb_calculate_qparams(ptr(mins), ptr(maxs), i32(DT[mins.dtype]), i64(mins.numel()), i32(qtype), i32(bits),
                                      i32(int(symmetric)), ptr(gs), ptr(scale), ptr(zp), i32(DT[zp_dtype]), stream_of(mins)))
    return scale, zp


def generate_gparam(mn, mx):
    """helpers.py:414 generate_gparam on device -> fp32 [1]."""
    require_cuda(mn, mx)
    mn, mx = _c(mn.reshape(1)), _c(mx.reshape(1))
    out = torch.empty(1, dtype=torch.float32, device=mn.device)
    check(lib().ctb_generate_gparam(ptr(mn), ptr(mx), i32(DT[mn.dtype]), ptr(out), stream_of(mn)))
    return out


def mxfp4_round_pow2(x):
    """quantization/utils/mxfp4_utils.py:43 round_to_power_2 (bf16 in, bf16 out)."""
    require_cuda(x)
    if x.dtype is not torch.bfloat16:
        raise AssertionError("round_to_power_2 takes bfloat16")
    x = _c(x)
    out = torch.empty_like(x)
    check(lib().ctb_mxfp4_round_pow2(ptr(x), i64(x.numel()), ptr(out), stream_of(x)))
    return out


def mxfp4_generate_scales(x):
    """quantization/utils/mxfp4_utils.py:75 generate_mxfp4_scales (bf16 in, uint8 exponents out)."""
    require_cuda(x)
    if x.dtype is not torch.bfloat16:
        raise AssertionError("generate_mxfp4_scales takes bfloat16")
    x = _c(x)
    out = torch.empty(x.shape, dtype=torch.uint8, device=x.device)
    check(lib().ctb_mxfp4_generate_scales(ptr(x), i64(x.numel()), ptr(out), stream_of(x)))
    return out


def mxfp4_convert_scales(scale, dtype=torch.bfloat16):
    """quantization/utils/mxfp4_utils.py:25 convert_mxfp4_exp_scale (uint8 exponents in, dense powers of two out)."""
    require_cuda(scale)
    if scale.dtype is not torch.uint8:
        raise AssertionError("mxfp4 scales are uint8 exponents")
    scale = _c(scale)
    out = torch.empty(scale.shape, dtype=dtype, device=scale.device)
    check(lib().ctb_mxfp4_convert_scales(ptr(scale), i64(scale.numel()), i32(DT[dtype]), ptr(out), stream_of(scale)))
    return out


def pack_int32(value, bits, packed_dim=1):
    """compressors/quantized_compressors/pack_quantized.py:186 pack_to_int32 (strides honoured, so a
    transposed view packs along dim 0 without a copy)."""
    require_cuda(value)
    if value.dtype is not torch.int8:
        raise ValueError("Tensor must be quantized to torch.int8 before packing")
    if bits > 8:
        raise ValueError("Packing is only supported for less than 8 bits")
    if bits < 1:
        raise ValueError(f"num_bits must be at least 1, got {bits}")
    v = value.transpose(0, 1) if packed_dim == 0 else value
    rows, cols = v.shape
    pf = 32 // bits
    out = torch.empty((rows, (cols + pf - 1) // pf), dtype=torch.int32, device=value.device)
    check(lib().ctb_pack_int32(ptr(v), i64(rows), i64(cols), i64(v.stride(0)), i64(v.stride(1)), i32(bits), ptr(out), stream_of(value)))
    return out.transpose(0, 1) if packed_dim == 0 else out


def unpack_int32(words, bits, shape, packed_dim=1):
    """pack_quantized.py:249 unpack_from_int32."""
    require_cuda(words)
    if words.dtype is not torch.int32:
        raise ValueError(f"Expected {torch.int32} but got {words.dtype}, Aborting unpack.")
    if bits > 8:
        raise ValueError("Unpacking is only supported for less than 8 bits")
    w = words.transpose(0, 1) if packed_dim == 0 else words
    rows = w.shape[0]
    cols = int(shape[0] if packed_dim == 0 else shape[1])
    out = torch.empty((rows, cols), dtype=torch.int8, device=words.device)
    check(lib().ctb_unpack_int32(ptr(w), i64(rows), i64(cols), i64(w.stride(0)), i64(w.stride(1)), i32(bits), ptr(out), stream_of(words)))
    return out.transpose(0, 1) if packed_dim == 0 else out


def pack_fp4(x):
    """compressors/quantized_compressors/fp4_quantized.py:136 pack_fp4_to_uint8."""
    require_cuda(x)
    x = _c(x)
    m, n = x.shape
    if n % 2 != 0:
        raise ValueError("tensor must have an even number of columns for nvfp4 compression")
    out = torch.empty((m, n // 2), dtype=torch.uint8, device=x.device)
    check(lib().ctb_pack_fp4(ptr(x), i32(DT[x.dtype]), i64(m), i64(n), ptr(out), stream_of(x)))
    return out


def unpack_fp4(a, m, n, dtype=torch.bfloat16):
    """fp4_quantized.py:188 unpack_fp4_from_uint8."""
    require_cuda(a)
    assert a.dtype == torch.uint8
    a = _c(a)
    out = torch.empty((m, n), dtype=dtype, device=a.device)
    check(lib().ctb_unpack_fp4(ptr(a), i64(m), i64(n), ptr(out), i32(DT[dtype]), stream_of(a)))
    return out


def pack_bitmasks(bytemasks):
    """utils/helpers.py:302 pack_bitmasks."""
    require_cuda(bytemasks)
    bm = _c(bytemasks).view(torch.uint8) if bytemasks.dtype == torch.bool else _c(bytemasks.to(torch.uint8))
    cols = bm.shape[-1]
    rows = bm.numel() // cols if cols else 0
    out = torch.empty(tuple(bm.shape[:-1]) + ((cols + 7) // 8,), dtype=torch.uint8, device=bm.device)
    check(lib().ctb_pack_bitmasks(ptr(bm), i64(rows), i64(cols), ptr(out), stream_of(bm)))
    return out


def unpack_bitmasks(packed, shape):
    """utils/helpers.py:316 unpack_bitmasks -> bool tensor of `shape`."""
    require_cuda(packed)
    packed = _c(packed)
    cols = int(shape[-1])
    rows = 1
    for s in shape[:-1]:
        rows *= int(s)
    out = torch.empty(tuple(int(s) for s in shape), dtype=torch.uint8, device=packed.device)
    check(lib().ctb_unpack_bitmasks(ptr(packed), i64(rows), i64(cols), ptr(out), stream_of(packed)))
    return out.view(torch.bool)


def sparse24_mask(x):
    """compressors/sparse_compressors/sparse_24_bitmask.py:227 get_24_bytemasks."""
    require_cuda(x)
    x = _c(x)
    if x.numel() % 4 != 0:
        raise ValueError("Tensor size must be a multiple of 4 for TWO_FOUR sparsity")
    out = torch.empty(x.shape, dtype=torch.uint8, device=x.device)
    check(lib().ctb_sparse24_mask(ptr(x), i32(DT[x.dtype]), i64(x.numel()), ptr(out), stream_of(x)))
    return out.view(torch.bool)


def _bitmask_workspace(rows, cols, device):
    lib().ctb_bitmask_workspace_bytes.restype = ctypes.c_int64
    n = int(lib().ctb_bitmask_workspace_bytes(i64(rows), i64(cols)))
    return torch.empty(max(n, 16), dtype=torch.uint8, device=device)


def _masked_compress(x, mask, sync=True):
    rows, cols = x.shape
    values = torch.empty(x.numel(), dtype=x.dtype, device=x.device)
    bitmask = torch.empty((rows, (cols + 7) // 8), dtype=torch.uint8, device=x.device)
    row_offsets = torch.empty(rows, dtype=torch.int64, device=x.device)
    nnz = torch.empty(1, dtype=torch.int64, device=x.device)
    if mask is None:
        ws = _bitmask_workspace(rows, cols, x.device)
        check(lib().ctb_bitmask_compress(ptr(x), i32(DT[x.dtype]), i64(rows), i64(cols), ptr(values), ptr(bitmask),
                                         ptr(row_offsets), ptr(nnz), ptr(ws), stream_of(x)))
    else:
        m = _c(mask).view(torch.uint8)
        check(lib().ctb_masked_compress(ptr(x), ptr(m), i32(DT[x.dtype]), i64(rows), i64(cols), ptr(values), ptr(bitmask),
                                        ptr(row_offsets), ptr(nnz), stream_of(x)))
    if not sync:  # full-capacity values buffer and the device-side count: no host round trip
        return values, bitmask, row_offsets, nnz
    count = int(nnz.item())
    if count < 0:
        raise TimeoutError("a bounded wait inside the single-pass bitmask kernel gave up; its outputs are incomplete")
    return values[:count], bitmask, row_offsets


def sparse24_compress(x):
    """sparse_24_bitmask.py:162 sparse24_bitmask_compress -> (values [rows, cols/2], bitmask)."""
    require_cuda(x)
    x = _c(x)
    rows, cols = x.shape
    if x.numel() % 4 != 0:
        raise ValueError("Tensor size must be a multiple of 4 for TWO_FOUR sparsity")
    if cols % 8 == 0:
        values = torch.empty((rows, cols // 2), dtype=x.dtype, device=x.device)
        bitmask = torch.empty((rows, cols // 8), dtype=torch.uint8, device=x.device)
        check(lib().ctb_sparse24_compress(ptr(x), i32(DT[x.dtype]), i64(rows), i64(cols), ptr(values), ptr(bitmask), stream_of(x)))
        return values, bitmask
    values, bitmask, _ = _masked_compress(x, sparse24_mask(x))
    return values.reshape(rows, cols // 2), bitmask


def quantize_fp8_sparse24(x, scale, zero_point=None):
    """Per-channel FP8 quantization (forward.py:462 _quantize to float8_e4m3fn) and sparse_24_bitmask.py:162
    sparse24_bitmask_compress of the result in one pass -> (values e4m3 [rows, cols/2], bitmask).
    x bf16 [rows, cols] with cols % 8 == 0, scale (bf16) and zero_point with one entry per row."""
    require_cuda(x, scale)
    x, scale = _c(x), _c(scale)
    if zero_point is not None:
        require_cuda(zero_point)
        zero_point = _c(zero_point)
        if zero_point.numel() != x.shape[0] or zero_point.dtype not in DT:
            raise ValueError("zero_point needs one entry per row in a supported dtype")
    if x.dtype != torch.bfloat16 or scale.dtype != torch.bfloat16 or x.dim() != 2:
        raise TypeError("quantize_fp8_sparse24 takes a 2-D bf16 tensor and bf16 scales")
    rows, cols = x.shape
    if scale.numel() != rows:
        raise ValueError(f"one scale per row expected, got {scale.numel()} for {rows} rows")
    values = torch.empty((rows, cols // 2), dtype=torch.float8_e4m3fn, device=x.device)
    bitmask = torch.empty((rows, cols // 8), dtype=torch.uint8, device=x.device)
    check(lib().ctb_quantize_fp8_sparse24(ptr(x), ptr(scale), ptr(zero_point), i32(DT[zero_point.dtype] if zero_point is not None else 0),
                                          i64(rows), i64(cols),
                                          ptr(values), ptr(bitmask), stream_of(x)))
    return values, bitmask


def bitmask_compress(x):
    """compressors/sparse_compressors/sparse_bitmask.py:131 bitmask_compress
    -> (values [nnz], bitmask [rows, ceil(cols/8)], row_offsets int64 [rows])."""
    require_cuda(x)
    return _masked_compress(_c(x), None)


def bitmask_decompress(values, bitmask, shape):
    """sparse_bitmask.py:152 bitmask_decompress / sparse_24_bitmask.py:206."""
    require_cuda(values, bitmask)
    values, bitmask = _c(values.flatten()), _c(bitmask)
    rows, cols = int(shape[0]), int(shape[1])
    out = torch.empty((rows, cols), dtype=values.dtype, device=bitmask.device)
    if values.numel() == 0:  # an all-zero tensor compresses to no values at all: nothing to read
        return out.zero_()
    ws = _bitmask_workspace(rows, cols, bitmask.device)
    check(lib().ctb_bitmask_decompress(ptr(values), ptr(bitmask), i32(DT[values.dtype]), i64(rows), i64(cols), ptr(out), ptr(ws),
                                       stream_of(bitmask)))
    return out


def sparse24_decompress(values, bitmask, shape):
    """sparse_24_bitmask.py:206 sparse24_bitmask_decompress (scan-free when the mask is two-per-four)."""
    require_cuda(values, bitmask)
    values, bitmask = _c(values.flatten()), _c(bitmask)
    rows, cols = int(shape[0]), int(shape[1])
    out = torch.empty((rows, cols), dtype=values.dtype, device=bitmask.device)
    if values.numel() == 0:  # an all-zero tensor compresses to no values at all: nothing to read
        return out.zero_()
    ws = _bitmask_workspace(rows, cols, bitmask.device)
    check(lib().ctb_sparse24_decompress(ptr(values), i64(values.numel()), ptr(bitmask), i32(DT[values.dtype]), i64(rows), i64(cols),
                                        ptr(out), ptr(ws), stream_of(bitmask)))
    return out


def sparse24_decompress_dequantize_fp8(values, bitmask, scale, shape):
    """sparse_24_bitmask.py:206 sparse24_bitmask_decompress of kept e4m3 values followed by the per-channel dequantize
    of forward.py:504 (bf16 scale, one per row, no zero point), in one pass -> bf16 [rows, cols]."""
    require_cuda(values, bitmask, scale)
    values, bitmask, scale = _c(values.flatten()), _c(bitmask), _c(scale)
    rows, cols = int(shape[0]), int(shape[1])
    if values.dtype != torch.float8_e4m3fn or scale.dtype != torch.bfloat16:
        raise TypeError("sparse24_decompress_dequantize_fp8 takes e4m3 values and bf16 scales")
    if scale.numel() != rows:
        raise ValueError(f"one scale per row expected, got {scale.numel()} for {rows} rows")
    out = torch.empty((rows, cols), dtype=torch.bfloat16, device=bitmask.device)
    if rows == 0 or cols == 0:
        return out
    lib().ctb_sparse24_dequantize_workspace_bytes.restype = ctypes.c_int64
    ws = torch.empty(int(lib().ctb_sparse24_dequantize_workspace_bytes(i64(rows), i64(cols))), dtype=torch.uint8, device=bitmask.device)
    check(lib().ctb_sparse24_decompress_dequantize_fp8(ptr(values), i64(values.numel()), ptr(bitmask), ptr(scale), i64(rows), i64(cols),
                                                       ptr(out), ptr(ws), stream_of(bitmask)))
    return out


def cutlass24_compress(dense):
    """utils/semi_structured_conversions.py:79 sparse_semi_structured_from_dense_cutlass for f16 / bf16 values or
    int8 codes -> (sparse [rows, cols/2], meta int16 [rows, cols/16] in CUTLASS's reordered layout)."""
    require_cuda(dense)
    if dense.dim() != 2:
        raise RuntimeError(f"Expected 2-dimensional dense tensor, got {dense.dim()}-dimensional tensor")
    dense = _c(dense)
    rows, cols = dense.shape
    sparse = torch.empty((rows, cols // 2), dtype=dense.dtype, device=dense.device)
    meta = torch.empty((rows, cols // 16), dtype=torch.int16, device=dense.device)
    check(lib().ctb_cutlass24_compress(ptr(dense), i32(DT[dense.dtype]), i64(rows), i64(cols), ptr(sparse), ptr(meta), stream_of(dense)))
    return sparse, meta


def cutlass24_decompress(sparse, meta):
    """utils/semi_structured_conversions.py:216 sparse_semi_structured_to_dense_cutlass (int16 reordered meta)."""
    require_cuda(sparse, meta)
    if sparse.dim() != 2 or meta.dim() != 2:
        raise RuntimeError("Expected 2-dimensional sparse and meta tensors")
    if meta.dtype is not torch.int16:
        raise RuntimeError(f"Invalid datatype {meta.dtype} of meta matrix")
    sparse, meta = _c(sparse), _c(meta)
    rows, k2 = sparse.shape
    if meta.shape[0] != rows or meta.shape[1] * 8 != k2:
        raise RuntimeError(f"meta matrix of shape {tuple(meta.shape)} does not match sparse matrix of shape {tuple(sparse.shape)}")
    dense = torch.empty((rows, 2 * k2), dtype=sparse.dtype, device=sparse.device)
    check(lib().ctb_cutlass24_decompress(ptr(sparse), ptr(meta), i32(DT[sparse.dtype]), i64(rows), i64(k2), ptr(dense), stream_of(sparse)))
    return dense


def marlin24_pack_weight(sparse, num_bits):
    """marlin_24.py:186-249: int8 codes [size_n, size_k] of the 2:4-compacted weight -> Marlin-24 packed int32
    [size_k/16, size_n*16/(32/num_bits)] (transpose, shift to unsigned, tile permutation, packing)."""
    require_cuda(sparse)
    sparse = _c(sparse.to(torch.int8))
    n, k2 = sparse.shape
    out = torch.empty((k2 // 16, n * 16 // (32 // num_bits)), dtype=torch.int32, device=sparse.device)
    check(lib().ctb_marlin24_pack_weight(ptr(sparse), i64(n), i64(k2), i32(num_bits), ptr(out), stream_of(sparse)))
    return out


def marlin24_pack_scales(scale, grouped):
    """marlin_24.py:252-273 (with the transpose of :188): fp16 scales [size_n, groups] -> [groups, size_n]."""
    require_cuda(scale)
    scale = _c(scale)
    if scale.element_size() != 2:
        raise ValueError("Marlin-24 scales are float16")
    n, g = scale.shape
    out = torch.empty((g, n), dtype=scale.dtype, device=scale.device)
    check(lib().ctb_marlin24_pack_scales(ptr(scale), i64(n), i64(g), i32(1 if grouped else 0), ptr(out), stream_of(scale)))
    return out


def hadamard(x, n, signs=None, inverse=False, side=0, precision=torch.float64, normalize=True):
    """transform/factory/hadamard.py:104 HadamardTransform.forward for a Linear weight
    (side 0 = weight_input, 1 = weight_output)."""
    require_cuda(x, signs)
    x = _c(x)
    rows, cols = x.shape
    s = None if signs is None else _c(signs.to(torch.int8))
    out = torch.empty_like(x)
    check(lib().ctb_hadamard(ptr(x), i32(DT[x.dtype]), i64(rows), i64(cols), i32(n), ptr(s), i32(int(inverse)), i32(side),
                             i32(_precision_code(precision)), i32(int(normalize)), ptr(out), stream_of(x)))
    return out


def absmax_quantize(x, *, qtype, bits, col_group, codec="pack32", out_dtype=None, global_scale=None,
                    hadamard_n=0, signs=None, precision=torch.float64):
    """Fused symmetric min-max calibration + quantize (+ pack), optionally with the weight_input
    Hadamard rotation in front.  Returns (quantized, scale)."""
    require_cuda(x, signs)
    x = _c(x)
    cols = x.shape[-1]
    rows = x.numel() // cols
    fp4 = qtype == QFLOAT and bits == 4
    sdt = torch.float8_e4m3fn if fp4 else x.dtype
    scale = torch.empty(tuple(x.shape[:-1]) + (cols // col_group,), dtype=sdt, device=x.device)
    if codec == "pack32":
        out = torch.empty(_packed_shape(x.shape, cols, codec, bits), dtype=torch.int32, device=x.device)
    elif codec == "fp4x2":
        out = torch.empty(_packed_shape(x.shape, cols, codec, bits), dtype=torch.uint8, device=x.device)
    else:
        out = torch.empty(x.shape, dtype=out_dtype, device=x.device)
    d = _desc(rows, cols, col_group, 1, cols // col_group, qtype, bits, x.dtype, scale, None, out_dtype, codec)
    gs = _gs(global_scale, x)
    s = None if signs is None else _c(signs.to(torch.int8))
    check(lib().ctb_absmax_quantize(ctypes.byref(d), ptr(x), ptr(gs), ptr(scale), ptr(out), i32(hadamard_n), ptr(s),
                                    i32(_precision_code(precision)), stream_of(x)))
    return out, scale


def tensor_table(ins, outs, scales, shapes):
    """A ctypes array of ``ctb_tensor_ref`` for the whole-shard entry points.  Build it once per shard and
    reuse it: the batched calls then cost one launch and no per-tensor Python work."""
    n = len(ins)
    table = (L.TensorRef * n)()
    for i in range(n):
        require_cuda(ins[i], outs[i], scales[i])
        table[i] = L.TensorRef(ins[i].data_ptr(), outs[i].data_ptr(), scales[i].data_ptr(), int(shapes[i][0]), int(shapes[i][1]))
    return table


def rotate_quantize_int4_batch(table, signs, precision=torch.float64, device=None, status=None):
    """Block-128 Hadamard rotation + symmetric int4 group-128 calibrate + quantize + pack of every tensor in
    `table` (weights bf16 in, int32 words and bf16 scales out), as one launch."""
    s = None if signs is None else signs
    stream = ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)
    check(lib().ctb_rotate_quantize_int4_batch(table, i32(len(table)), ptr(s), i32(_precision_code(precision)), ptr(status), stream))


def rotate_quantize_int4_batch_bounded(table, signs, status, spin_cycles, skip_tile=-1, device=None):
    """The tensor-core form of rotate_quantize_int4_batch with the bound of its device-side waits given in SM clocks
    and, for skip_tile >= 0, with that tile's copy left out so that the wait for it runs out.  Exercises the kernel's
    error path: it returns, and `status` (device int32) then reads 5 (CTB_ETIMEOUT)."""
    stream = ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)
    check(lib().ctb_rotate_quantize_int4_batch_bounded(table, i32(len(table)), ptr(signs), ptr(status), i64(spin_cycles), i32(skip_tile), stream))


def quantize_pack_int4_batch(table, device=None):
    """quantize with the GIVEN bf16 scales (symmetric int4, group 128) + pack_to_int32 of every tensor in `table`
    (weights in, words out, scales read), as one launch."""
    stream = ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)
    check(lib().ctb_quantize_pack_int4_batch(table, i32(len(table)), stream))


def quantize_fp8_channel_batch(table, zero_points=None, device=None):
    """Per-channel FP8 quantize (static bf16 scale, one per row) of every tensor in `table` (bf16 weights in, e4m3 out,
    scales read), as one launch.  zero_points: None, or one tensor / None per table entry."""
    stream = ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)
    zps, zdt = None, 0
    if zero_points is not None and any(z is not None for z in zero_points):
        dts = {z.dtype for z in zero_points if z is not None}
        if len(dts) != 1 or next(iter(dts)) not in DT:
            raise TypeError("zero points of one call must share one supported dtype")
        zdt = DT[next(iter(dts))]
        zps = (ctypes.c_void_p * len(table))(*[None if z is None else z.data_ptr() for z in zero_points])
    check(lib().ctb_quantize_fp8_channel_batch(table, i32(len(table)), zps, i32(zdt), stream))


def dequantize_fp8_channel_batch(table, device=None):
    """dequantize (e4m3 codes, static bf16 scale per row, no zero point) of every tensor in `table` (codes in, bf16
    weights out), as one launch."""
    stream = ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)
    check(lib().ctb_dequantize_fp8_channel_batch(table, i32(len(table)), stream))


def _pointer_array(tensors):
    return (ctypes.c_void_p * len(tensors))(*[None if t is None else t.data_ptr() for t in tensors])


def quantize_fp4_g16_batch(table, global_scales, zero_points=None, device=None):
    """NVFP4 quantize + pack (e4m3 group-16 scales, fp32 global scale per tensor) of every tensor in `table` (bf16
    weights in, uint8 pairs of e2m1 codes out, scales read), as one launch."""
    stream = ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)
    zps, zdt = None, 0
    if zero_points is not None and any(z is not None for z in zero_points):
        dts = {z.dtype for z in zero_points if z is not None}
        if len(dts) != 1 or next(iter(dts)) not in DT:
            raise TypeError("zero points of one call must share one supported dtype")
        zdt, zps = DT[next(iter(dts))], _pointer_array(zero_points)
    check(lib().ctb_quantize_fp4_g16_batch(table, i32(len(global_scales)), _pointer_array(global_scales), zps, i32(zdt), stream))


def dequantize_fp4_g16_batch(table, global_scales, device=None):
    """unpack + dequantize NVFP4 (e4m3 group-16 scales, fp32 global scale, no zero point) of every tensor in `table`
    (uint8 code pairs in, bf16 weights out), as one launch."""
    stream = ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)
    check(lib().ctb_dequantize_fp4_g16_batch(table, i32(len(global_scales)), _pointer_array(global_scales), stream))


def unpack_dequantize_int4_batch(table, device=None):
    """unpack_from_int32 + dequantize (int4, group 128, bf16 scales, symmetric) of every tensor in `table`
    (words in, bf16 weights out), as one launch."""
    stream = ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)
    check(lib().ctb_unpack_dequantize_int4_batch(table, i32(len(table)), stream))
