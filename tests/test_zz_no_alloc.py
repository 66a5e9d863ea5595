"""The decompress entry point that brings its own scratch (`ctb_bitmask_decompress_static`) must give
exactly what `ctb_bitmask_decompress` gives.  It exists for hosts that may not allocate device memory
at decompress time (fixed-arena servers, load hooks), so the test drives the C ABI directly with
buffers allocated up front, twice in a row because the library-owned scratch keeps the previous
call's contents.  Collected last on purpose."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _call(fn, values, bitmask, rows, cols, out, *extra):
    from compressed_tensors_b200 import _lib as L

    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    return fn(L.ptr(values), L.ptr(bitmask), L.i32(L.DT[values.dtype]), L.i64(rows), L.i64(cols), L.ptr(out), *extra, stream)


def test_static_scratch_decompress_matches_twice():
    from compressed_tensors_b200 import _lib as L
    from compressed_tensors_b200 import ops

    lib = L.lib()
    g = torch.Generator().manual_seed(11)
    for rows, cols, dtype in ((300, 1000, torch.bfloat16), (64, 4096, torch.float32)):
        for rep in range(2):  # two different inputs back to back: stale scratch must not leak through
            x = torch.randn(rows, cols, generator=g)
            x[torch.rand(rows, cols, generator=g) < 0.5 + 0.2 * rep] = 0
            x = x.to(dtype).cuda()
            values, bitmask, _ = ops.bitmask_compress(x)
            want = torch.empty_like(x)
            lib.ctb_bitmask_workspace_bytes.restype = ctypes.c_int64
            ws = torch.empty(int(lib.ctb_bitmask_workspace_bytes(L.i64(rows), L.i64(cols))), dtype=torch.uint8, device="cuda")
            got = torch.full_like(x, 7.0)
            assert _call(lib.ctb_bitmask_decompress, values, bitmask, rows, cols, want, L.ptr(ws)) == 0
            assert _call(lib.ctb_bitmask_decompress_static, values, bitmask, rows, cols, got) == 0
            torch.cuda.synchronize()
            # the point of the entry point: once its first call on the device is behind it, a call takes no device
            # memory, neither from the driver nor from torch's allocator
            free0, _ = torch.cuda.mem_get_info()
            allocs0 = torch.cuda.memory_stats()["allocation.all.allocated"]
            assert _call(lib.ctb_bitmask_decompress_static, values, bitmask, rows, cols, got) == 0
            torch.cuda.synchronize()
            assert torch.cuda.mem_get_info()[0] == free0
            assert torch.cuda.memory_stats()["allocation.all.allocated"] == allocs0
            assert torch.equal(got.view(torch.uint8), want.view(torch.uint8))
            assert torch.equal(got, torch.where(x == 0, torch.zeros_like(x), x))


def test_static_scratch_rejects_too_many_rows():
    from compressed_tensors_b200 import _lib as L

    lib = L.lib()
    rows, cols = 65537, 8
    values = torch.zeros(8, dtype=torch.bfloat16, device="cuda")
    bitmask = torch.zeros((rows, 1), dtype=torch.uint8, device="cuda")
    out = torch.empty((rows, cols), dtype=torch.bfloat16, device="cuda")
    rc = _call(lib.ctb_bitmask_decompress_static, values, bitmask, rows, cols, out)
    assert rc == 1  # CTB_EINVAL_SHAPE
    assert b"65536" in lib.ctb_last_error_string()
