"""ctypes front end of the CPU oracle (``libctb_oracle.so``).

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, by the smoke check and by the CPU-baseline
leg of the benchmark.  Nothing in the shipped package may import this module.

torch CPU tensors are used purely as typed buffers (numpy has no bfloat16 / float8); all
arithmetic happens in the C code.
"""
import ctypes
import os
import subprocess

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libctb_oracle.so")

DT = {
    torch.bfloat16: 0,
    torch.float16: 1,
    torch.float32: 2,
    torch.float64: 3,
    torch.int8: 4,
    torch.float8_e4m3fn: 5,
    torch.uint8: 6,
    torch.bool: 6,
    torch.int32: 7,
    torch.int64: 8,
}
QINT, QFLOAT = 0, 1


def build(force: bool = False) -> str:
    """Compile the oracle with the recipe in ``oracle/Makefile``."""
    srcs = [os.path.join(_HERE, f) for f in ("ctb_oracle.c", "sparse24_topk.cpp", "Makefile")]
    stale = not os.path.exists(_LIB_PATH) or any(
        os.path.getmtime(s) > os.path.getmtime(_LIB_PATH) for s in srcs
    )
    if force or stale:
        subprocess.run(["make", "-C", _HERE, "-B"], check=True, capture_output=True)
    return _LIB_PATH


class _Desc(ctypes.Structure):
    _fields_ = [
        ("rows", ctypes.c_int64),
        ("cols", ctypes.c_int64),
        ("col_group", ctypes.c_int64),
        ("row_group", ctypes.c_int64),
        ("scale_row_stride", ctypes.c_int64),
        ("qtype", ctypes.c_int32),
        ("bits", ctypes.c_int32),
        ("x_dtype", ctypes.c_int32),
        ("scale_dtype", ctypes.c_int32),
        ("zp_dtype", ctypes.c_int32),
        ("out_dtype", ctypes.c_int32),
    ]


_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        _lib = ctypes.CDLL(_LIB_PATH)
        _lib.orc_generate_gparam.restype = ctypes.c_float
        _lib.orc_bitmask_compress.restype = ctypes.c_int64
    return _lib


def set_threads(n: int) -> None:
    """OpenMP thread count for the oracle (used by the timed CPU baseline)."""
    omp = ctypes.CDLL("libgomp.so.1")
    omp.omp_set_num_threads(int(n))


def _p(t):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _c(t):
    assert t.device.type == "cpu"
    return t.contiguous()


def _qdq(mode, x, scale, zp, *, qtype, bits, col_group, row_group, scale_row_stride, out_dtype,
         g_idx=None, global_scale=None):
    x, scale = _c(x), _c(scale)
    zp = None if zp is None else _c(zp)
    g_idx = None if g_idx is None else _c(g_idx.to(torch.int32))
    gs = None if global_scale is None else _c(global_scale.to(torch.float32))
    cols = x.shape[-1]
    rows = x.numel() // cols
    d = _Desc(rows, cols, col_group, row_group, scale_row_stride, qtype, bits, DT[x.dtype],
              DT[scale.dtype], DT[zp.dtype] if zp is not None else 0, DT[out_dtype])
    out = torch.empty(x.shape, dtype=out_dtype)
    rc = lib().orc_qdq(ctypes.byref(d), mode, _p(x), _p(scale), _p(zp), _p(g_idx), _p(gs), _p(out))
    assert rc == 0
    return out


def quantize(x, scale, zp=None, **kw):
    return _qdq(0, x, scale, zp, **kw)


def dequantize(xq, scale, zp=None, **kw):
    return _qdq(1, xq, scale, zp, **kw)


def fake_quantize(x, scale, zp=None, **kw):
    return _qdq(2, x, scale, zp, **kw)


def minmax(x, row_group, col_group):
    x = _c(x)
    cols = x.shape[-1]
    rows = x.numel() // cols
    shape = (rows // row_group, cols // col_group)
    mn = torch.empty(shape, dtype=x.dtype)
    mx = torch.empty(shape, dtype=x.dtype)
    lib().orc_minmax(_p(x), DT[x.dtype], ctypes.c_int64(rows), ctypes.c_int64(cols),
                     ctypes.c_int64(row_group), ctypes.c_int64(col_group), _p(mn), _p(mx))
    return mn, mx


def calculate_qparams(mins, maxs, *, qtype, bits, symmetric, global_scale=None):
    mins, maxs = _c(mins), _c(maxs)
    fp4 = qtype == QFLOAT and bits == 4
    zp_dtype = torch.int8 if qtype == QINT else torch.float8_e4m3fn
    sdt = torch.float8_e4m3fn if (fp4 and global_scale is not None) else mins.dtype
    scale = torch.empty(mins.shape, dtype=sdt)
    zp = torch.empty(mins.shape, dtype=zp_dtype)
    gs = None if global_scale is None else _c(global_scale.to(torch.float32))
    rc = lib().orc_calculate_qparams(_p(mins), _p(maxs), DT[mins.dtype], ctypes.c_int64(mins.numel()),
                                     qtype, bits, int(symmetric), _p(gs), _p(scale), _p(zp), DT[zp_dtype])
    assert rc == 0
    return scale, zp


def generate_gparam(mn, mx):
    mn, mx = _c(mn.reshape(1)), _c(mx.reshape(1))
    return torch.tensor([lib().orc_generate_gparam(_p(mn), _p(mx), DT[mn.dtype])], dtype=torch.float32)


def pack_int32(q, bits):
    q = _c(q)
    rows, cols = q.shape
    pf = 32 // bits
    out = torch.empty((rows, (cols + pf - 1) // pf), dtype=torch.int32)
    lib().orc_pack_int32(_p(q), ctypes.c_int64(rows), ctypes.c_int64(cols), bits, _p(out))
    return out


def unpack_int32(w, bits, shape):
    w = _c(w)
    rows, cols = shape
    out = torch.empty((rows, cols), dtype=torch.int8)
    lib().orc_unpack_int32(_p(w), ctypes.c_int64(rows), ctypes.c_int64(cols), bits, _p(out))
    return out


def pack_fp4(x):
    x = _c(x)
    m, n = x.shape
    out = torch.empty((m, n // 2), dtype=torch.uint8)
    rc = lib().orc_pack_fp4(_p(x), DT[x.dtype], ctypes.c_int64(m), ctypes.c_int64(n), _p(out))
    if rc:
        raise ValueError("odd column count")
    return out


def unpack_fp4(a, m, n, dtype=torch.bfloat16):
    a = _c(a)
    out = torch.empty((m, n), dtype=dtype)
    lib().orc_unpack_fp4(_p(a), ctypes.c_int64(m), ctypes.c_int64(n), _p(out), DT[dtype])
    return out


def pack_bitmasks(bytemask):
    bm = _c(bytemask.to(torch.uint8))
    rows, cols = bm.shape
    out = torch.empty((rows, (cols + 7) // 8), dtype=torch.uint8)
    lib().orc_pack_bitmasks(_p(bm), ctypes.c_int64(rows), ctypes.c_int64(cols), _p(out))
    return out


def unpack_bitmasks(packed, shape):
    packed = _c(packed)
    rows, cols = shape
    out = torch.empty((rows, cols), dtype=torch.uint8)
    lib().orc_unpack_bitmasks(_p(packed), ctypes.c_int64(rows), ctypes.c_int64(cols), _p(out))
    return out.bool()


def bitmask_compress(x):
    x = _c(x)
    rows, cols = x.shape
    values = torch.empty(x.numel(), dtype=x.dtype)
    bitmask = torch.empty((rows, (cols + 7) // 8), dtype=torch.uint8)
    row_offsets = torch.empty(rows, dtype=torch.int64)
    nnz = lib().orc_bitmask_compress(_p(x), DT[x.dtype], ctypes.c_int64(rows), ctypes.c_int64(cols),
                                     _p(values), _p(bitmask), _p(row_offsets))
    return values[:nnz].clone(), bitmask, row_offsets


def bitmask_decompress(values, bitmask, shape):
    values, bitmask = _c(values.flatten()), _c(bitmask)
    rows, cols = shape
    out = torch.empty((rows, cols), dtype=values.dtype)
    lib().orc_bitmask_decompress(_p(values), _p(bitmask), DT[values.dtype], ctypes.c_int64(rows),
                                 ctypes.c_int64(cols), _p(out))
    return out


def sparse24_mask(x):
    x = _c(x)
    out = torch.empty(x.shape, dtype=torch.uint8)
    rc = lib().orc_sparse24_mask(_p(x), DT[x.dtype], ctypes.c_int64(x.numel()), _p(out))
    if rc:
        raise ValueError("numel % 4")
    return out.bool()


def sparse24_compress(x):
    x = _c(x)
    rows, cols = x.shape
    mask = _c(sparse24_mask(x).to(torch.uint8))
    values = torch.empty((rows, cols // 2), dtype=x.dtype)
    bitmask = torch.empty((rows, (cols + 7) // 8), dtype=torch.uint8)
    rc = lib().orc_sparse24_gather(_p(x), DT[x.dtype], _p(mask), ctypes.c_int64(rows),
                                   ctypes.c_int64(cols), _p(values), _p(bitmask))
    assert rc == 0
    return values, bitmask


def cutlass24_compress(q):
    q = _c(q.to(torch.int8))
    m, k = q.shape
    sparse = torch.empty((m, k // 2), dtype=torch.int8)
    meta = torch.empty((m, k // 16), dtype=torch.int16)
    rc = lib().orc_cutlass24_compress(_p(q), ctypes.c_int64(m), ctypes.c_int64(k), _p(sparse), _p(meta))
    if rc:
        raise RuntimeError("rows must be divisible by 32 and columns by 16")
    return sparse, meta


def cutlass24_decompress(sparse, meta):
    sparse, meta = _c(sparse.to(torch.int8)), _c(meta)
    m, k2 = sparse.shape
    dense = torch.empty((m, 2 * k2), dtype=torch.int8)
    rc = lib().orc_cutlass24_decompress(_p(sparse), _p(meta), ctypes.c_int64(m), ctypes.c_int64(k2), _p(dense))
    assert rc == 0
    return dense


def marlin24_pack_weight(sparse, bits):
    sparse = _c(sparse.to(torch.int8))
    n, k2 = sparse.shape
    out = torch.empty((k2 // 16, n * 16 // (32 // bits)), dtype=torch.int32)
    rc = lib().orc_marlin24_pack_weight(_p(sparse), ctypes.c_int64(n), ctypes.c_int64(k2), bits, _p(out))
    assert rc == 0
    return out


def marlin24_pack_scales(scale, grouped):
    scale = _c(scale.to(torch.float16))
    n, g = scale.shape
    out = torch.empty((g, n), dtype=torch.float16)
    rc = lib().orc_marlin24_pack_scales(_p(scale), ctypes.c_int64(n), ctypes.c_int64(g), int(grouped), _p(out))
    assert rc == 0
    return out


def mxfp4_round_pow2(x):
    x = _c(x)
    out = torch.empty_like(x)
    lib().orc_mxfp4_round_pow2(_p(x), ctypes.c_int64(x.numel()), _p(out))
    return out


def mxfp4_generate_scales(x):
    x = _c(x)
    out = torch.empty(x.shape, dtype=torch.uint8)
    lib().orc_mxfp4_generate_scales(_p(x), ctypes.c_int64(x.numel()), _p(out))
    return out


def mxfp4_convert_scales(scale, dtype=torch.bfloat16):
    scale = _c(scale)
    out = torch.empty(scale.shape, dtype=dtype)
    lib().orc_mxfp4_convert_scales(_p(scale), ctypes.c_int64(scale.numel()), DT[dtype], _p(out))
    return out


def hadamard(x, n, signs=None, inverse=False, side=0):
    x = _c(x)
    rows, cols = x.shape
    s = None if signs is None else _c(signs.to(torch.int8))
    out = torch.empty_like(x)
    rc = lib().orc_hadamard(_p(x), DT[x.dtype], ctypes.c_int64(rows), ctypes.c_int64(cols),
                            ctypes.c_int64(n), _p(s), int(inverse), int(side), _p(out))
    if rc:
        raise ValueError("shape not divisible by the Hadamard size")
    return out
