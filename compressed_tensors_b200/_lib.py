"""ctypes binding of ``libctb200.so``.

There is no CPU fallback: if the library is missing or a tensor is not on a CUDA device the
call fails loudly.
"""
import ctypes
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libctb200.so")

# ctb_dtype codes (include/ctb200.h)
BF16, F16, F32, F64, I8, E4M3, U8, I32, I64 = range(9)
DT = {
    torch.bfloat16: BF16,
    torch.float16: F16,
    torch.float32: F32,
    torch.float64: F64,
    torch.int8: I8,
    torch.float8_e4m3fn: E4M3,
    torch.uint8: U8,
    torch.bool: U8,
    torch.int32: I32,
    torch.int64: I64,
}
QINT, QFLOAT = 0, 1
CODE_DTYPE, CODE_PACK32, CODE_FP4X2 = 0, 1, 2

# ctb_status -> exception type, mirroring what the reference raises for the same mistake
_STATUS_EXC = {
    1: ValueError,          # CTB_EINVAL_SHAPE
    2: TypeError,           # CTB_EINVAL_DTYPE
    3: ValueError,          # CTB_EINVAL_ALIGN
    4: ValueError,          # CTB_EINVAL_NULL
    5: TimeoutError,        # CTB_ETIMEOUT
    6: RuntimeError,        # CTB_ECUDA
    7: NotImplementedError, # CTB_EUNSUPPORTED
}


class QDesc(ctypes.Structure):
    """Mirror of ``ctb_qdesc``."""

    _fields_ = [
        ("rows", ctypes.c_int64),
        ("cols", ctypes.c_int64),
        ("col_group", ctypes.c_int64),
        ("row_group", ctypes.c_int64),
        ("scale_row_stride", ctypes.c_int64),
        ("qtype", ctypes.c_int32),
        ("num_bits", ctypes.c_int32),
        ("x_dtype", ctypes.c_int32),
        ("scale_dtype", ctypes.c_int32),
        ("zp_dtype", ctypes.c_int32),
        ("q_dtype", ctypes.c_int32),
        ("codec", ctypes.c_int32),
        ("reserved", ctypes.c_int32),
    ]


class TensorRef(ctypes.Structure):
    """Mirror of ``ctb_tensor_ref``."""

    _fields_ = [("inp", ctypes.c_void_p), ("out", ctypes.c_void_p), ("scale", ctypes.c_void_p),
                ("rows", ctypes.c_int64), ("cols", ctypes.c_int64)]


_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m compressed_tensors_b200._build`. "
                "This package has no CPU or eager fallback."
            )
        _lib = ctypes.CDLL(LIB_PATH)
        _lib.ctb_version.restype = ctypes.c_char_p
        _lib.ctb_last_error_string.restype = ctypes.c_char_p
        _lib.ctb_launch_count.restype = ctypes.c_int64
        _lib.ctb_minmax_workspace_bytes.restype = ctypes.c_int64
        _lib.ctb_minmax_workspace_bytes.argtypes = [ctypes.c_int64] * 4
    return _lib


def check(status: int) -> None:
    if status != 0:
        msg = lib().ctb_last_error_string().decode()
        raise _STATUS_EXC.get(status, RuntimeError)(msg)


def launch_count() -> int:
    return int(lib().ctb_launch_count())


def ptr(t):
    """Device pointer of a tensor (None -> NULL)."""
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def stream_of(t: torch.Tensor):
    return ctypes.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def require_cuda(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError(
                "compressed_tensors_b200 runs on CUDA tensors only (no CPU fallback); got a "
                f"{t.device} tensor"
            )


def i64(v) -> ctypes.c_int64:
    return ctypes.c_int64(int(v))


def i32(v) -> ctypes.c_int32:
    return ctypes.c_int32(int(v))


def on_gpu(t):
    """Host plumbing for callers that hand in CPU tensors (the reference's compressors accept any
    device): copy to the current CUDA device.  The arithmetic still runs only in the CUDA kernels."""
    if t is None or t.is_cuda:
        return t
    if not torch.cuda.is_available():
        raise RuntimeError("compressed_tensors_b200 needs a CUDA device (no CPU fallback)")
    return t.cuda()
