"""The SIMD formulation of the 2:4 keep rule (csrc/ctb_sparse24_simd.cuh), compiled for the host, against the
oracle's restatement of torch.topk on runs of four (sparse_24_bitmask.py:244-256).  No GPU needed: the header
is plain integer logic shared by the host build and the CUDA kernels."""
import ctypes
import itertools
import pathlib
import subprocess

import pytest
import torch

from oracle import ref

ROOT = pathlib.Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def simd(tmp_path_factory):
    so = tmp_path_factory.mktemp("simd24") / "libsimd24.so"
    subprocess.run(["/usr/bin/g++", "-O2", "-shared", "-fPIC", "-std=c++17", "-I", str(ROOT / "compressed_tensors_b200" / "csrc"),
                    str(ROOT / "tests" / "sparse24_simd_host.cpp"), "-o", str(so)], check=True)
    return ctypes.CDLL(str(so))


def _pack(simd, x):
    """x: 2-D tensor of an 8- or 16-bit dtype with cols % 16 == 0 -> (values, bitmask) from the SIMD host build."""
    rows, cols = x.shape
    x = x.contiguous()
    values = torch.empty((rows, cols // 2), dtype=x.dtype)
    bitmask = torch.empty((rows, cols // 8), dtype=torch.uint8)
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    if x.element_size() == 1:
        simd.simd24_pack_u8(p(x), ctypes.c_int64(x.numel() // 16), p(values), p(bitmask))
    else:
        simd.simd24_pack_u16(p(x), ctypes.c_int64(x.numel() // 8), p(values), p(bitmask))
    return values, bitmask


def _check(simd, x):
    v, b = _pack(simd, x)
    ov, ob = ref.sparse24_compress(x)
    assert torch.equal(b, ob)
    assert torch.equal(v.view(torch.uint8), ov.view(torch.uint8))
    # the bytemask form of the same rule (get_24_bytemasks)
    xc = x.contiguous()
    bm = torch.empty(xc.shape, dtype=torch.uint8)
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    if xc.element_size() == 1:
        simd.simd24_bytemask_u8(p(xc), ctypes.c_int64(xc.numel() // 16), p(bm))
    else:
        simd.simd24_bytemask_u16(p(xc), ctypes.c_int64(xc.numel() // 8), p(bm))
    assert torch.equal(bm.bool(), ref.sparse24_mask(x))


def _orderings(levels):
    """every assignment of `levels` to four slots, as rows of 16 elements (four runs per row)"""
    combos = list(itertools.product(levels, repeat=4))
    while len(combos) % 4:
        combos.append(combos[-1])
    return torch.tensor(combos).reshape(-1, 16)


def test_every_weak_ordering_int8(simd):
    # 7^4 assignments cover all 75 weak orderings, with the wrap-around value -128 (ranks below zero) among them
    x = _orderings([-128, -127, -3, 0, 3, 5, 127]).to(torch.int8)
    _check(simd, x)


def test_every_weak_ordering_bf16(simd):
    x = _orderings([-2.0, -0.5, -0.0, 0.0, 0.5, 1.0, 2.0]).to(torch.bfloat16)
    _check(simd, x)
    _check(simd, x.to(torch.float16))


def test_all_byte_pairs_e4m3(simd):
    # every pair of byte values meets in a run, next to two fixed neighbours (65536 runs)
    a = torch.arange(256, dtype=torch.int32)
    runs = torch.stack([a.repeat_interleave(256), a.repeat(256), torch.full((65536,), 0x38), torch.full((65536,), 0xB0)], dim=1)
    for perm in ([0, 1, 2, 3], [2, 0, 3, 1], [3, 2, 1, 0]):
        x = runs[:, perm].to(torch.uint8).reshape(-1, 16).view(torch.float8_e4m3fn)
        _check(simd, x)


def test_random(simd):
    g = torch.Generator().manual_seed(24)
    _check(simd, torch.randint(-128, 128, (512, 1024), generator=g, dtype=torch.int8))
    _check(simd, torch.randint(0, 256, (512, 1024), generator=g, dtype=torch.uint8).view(torch.float8_e4m3fn))
    _check(simd, torch.randint(-4, 5, (512, 1024), generator=g, dtype=torch.int8))  # many ties
    _check(simd, torch.randint(0, 65536, (256, 1024), generator=g, dtype=torch.int32).to(torch.uint16).view(torch.bfloat16))
    _check(simd, (torch.randint(-3, 4, (256, 1024), generator=g) * 0.25).to(torch.bfloat16))


def test_fastdiv_matches_integer_division(tmp_path):
    """csrc/ctb_fastdiv.h (the index arithmetic of the BLOCK-strategy kernels): every divisor up to 4096, powers of
    two and their neighbours, large divisors, on random 31-bit numerators and on the edges of every quotient step"""
    so = tmp_path / "libfastdiv.so"
    subprocess.run(["/usr/bin/g++", "-O2", "-shared", "-fPIC", "-std=c++17", "-I", str(ROOT / "compressed_tensors_b200" / "csrc"),
                    str(ROOT / "tests" / "fastdiv_host.cpp"), "-o", str(so)], check=True)
    lib = ctypes.CDLL(str(so))
    lib.fastdiv_mismatches.restype = ctypes.c_int64
    g = torch.Generator().manual_seed(5)
    ns = torch.randint(0, 2 ** 31, (4096,), generator=g, dtype=torch.int64).to(torch.int32).contiguous()
    divisors = list(range(1, 4097)) + [2 ** k + o for k in range(12, 31) for o in (-1, 0, 1)] + [2 ** 31 - 1, 1000003, 14336 // 8, 28672]
    for d in divisors:
        assert lib.fastdiv_mismatches(ctypes.c_uint32(d), ctypes.c_void_p(ns.data_ptr()), ctypes.c_int64(ns.numel())) == 0, d
