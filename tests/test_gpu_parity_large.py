"""Parity of the CUDA path against the CPU oracle on seeded inputs at sizes the oracle finishes in
seconds, plus size-independent properties at the benchmark's full tensor sizes."""
import itertools

import pytest
import torch

from tests.helpers import assert_bit_equal

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from compressed_tensors_b200 import ops as o
    return o


@pytest.fixture(scope="module")
def orc():
    from oracle import ref
    ref.build()
    return ref


def weights(rows, cols, seed=0, std=0.02):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(rows, cols, generator=g) * std).to(torch.bfloat16)


def signs128(seed=0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randint(0, 2, (128,), generator=g) * 2 - 1).to(torch.int8)


def oracle_w4(orc, w, group=128):
    mn, mx = orc.minmax(w, 1, group)
    scale, zp = orc.calculate_qparams(mn, mx, qtype=orc.QINT, bits=4, symmetric=True)
    kw = dict(qtype=orc.QINT, bits=4, col_group=group, row_group=1, scale_row_stride=w.shape[1] // group)
    words = orc.pack_int32(orc.quantize(w, scale, zp, out_dtype=torch.int8, **kw), 4)
    deq = orc.dequantize(orc.unpack_int32(words, 4, w.shape), scale, None, out_dtype=torch.bfloat16, **kw)
    return scale, words, deq


def test_w4a16_group128_matches_oracle(ops, orc):
    """BASELINE config 1 math on a 1024x4096 slice: scales, packed words and dequantized values bit-exact."""
    w = weights(1024, 4096)
    scale, words, deq = oracle_w4(orc, w)
    got_words, got_scale = ops.absmax_quantize(w.cuda(), qtype=ops.QINT, bits=4, col_group=128, codec="pack32")
    assert_bit_equal(got_scale.cpu(), scale, "scales")
    assert_bit_equal(got_words.cpu(), words, "packed words")
    given = ops.quantize(w.cuda(), scale.cuda(), None, qtype=ops.QINT, bits=4, col_group=128, scale_row_stride=32, codec="pack32")
    assert_bit_equal(given.cpu(), words, "packed words from given scales")
    got = ops.dequantize(got_words, got_scale, None, qtype=ops.QINT, bits=4, col_group=128, scale_row_stride=32,
                         out_dtype=torch.bfloat16, codec="pack32", cols=4096)
    assert_bit_equal(got.cpu(), deq, "dequantized")


def test_w4a16_asymmetric_matches_oracle(ops, orc):
    w = weights(256, 1024, seed=5) + 0.01
    w = w.to(torch.bfloat16)
    mn, mx = orc.minmax(w, 1, 128)
    scale, zp = orc.calculate_qparams(mn, mx, qtype=orc.QINT, bits=4, symmetric=False)
    kw = dict(qtype=orc.QINT, bits=4, col_group=128, row_group=1, scale_row_stride=8)
    words = orc.pack_int32(orc.quantize(w, scale, zp, out_dtype=torch.int8, **kw), 4)
    deq = orc.dequantize(orc.unpack_int32(words, 4, w.shape), scale, zp, out_dtype=torch.bfloat16, **kw)
    gw = ops.quantize(w.cuda(), scale.cuda(), zp.cuda(), codec="pack32", **{k: v for k, v in kw.items()})
    assert_bit_equal(gw.cpu(), words, "asymmetric packed words")
    gd = ops.dequantize(gw, scale.cuda(), zp.cuda(), out_dtype=torch.bfloat16, codec="pack32", cols=1024, **kw)
    assert_bit_equal(gd.cpu(), deq, "asymmetric dequantized")


def test_rotate_quantize_exact_mode_matches_oracle(ops, orc):
    """float64-accumulated rotation fused with int4 g128: bit-exact against rotate -> calibrate -> quantize -> pack."""
    w, sg = weights(512, 4096, seed=1), signs128(1)
    rot = orc.hadamard(w, 128, signs=sg)
    scale, words, _ = oracle_w4(orc, rot)
    assert_bit_equal(ops.hadamard(w.cuda(), 128, signs=sg.cuda(), precision=torch.float64).cpu(), rot, "rotated weights")
    gw, gs = ops.absmax_quantize(w.cuda(), qtype=ops.QINT, bits=4, col_group=128, codec="pack32", hadamard_n=128,
                                 signs=sg.cuda(), precision=torch.float64)
    assert_bit_equal(gs.cpu(), scale, "scales")
    assert_bit_equal(gw.cpu(), words, "packed words")


@pytest.mark.parametrize("mode", ["float32", "tensor"])
def test_rotate_quantize_fast_modes_staged(ops, orc, mode):
    """fp32-accumulated rotation: the float32 butterfly and the tcgen05 tensor-core GEMM (bf16 operands, fp32
    accumulators in TMEM).  Stage 1: rotated weights within the stated tolerance of the float64 result (norm-wise
    rel-err <= 1e-3, all but a few parts per million identical, none off by more than 4 bf16 steps).  Stage 2: the
    fused kernel equals the ORACLE's calibrate+quantize+pack applied to that rotated tensor, bit for bit."""
    from tests.helpers import bf16_ulp_distance

    precision = torch.float32 if mode == "float32" else ops.ROT_TENSOR
    w, sg = weights(512, 4096, seed=2), signs128(2)
    exact = orc.hadamard(w, 128, signs=sg)
    fast = ops.hadamard(w.cuda(), 128, signs=sg.cuda(), precision=precision).cpu()
    err = (fast.double() - exact.double()).norm() / exact.double().norm()
    assert err <= 1e-3, float(err)
    differ = (fast.view(torch.int16) != exact.view(torch.int16)).sum().item()
    assert differ <= 50e-6 * exact.numel(), differ
    assert bf16_ulp_distance(fast, exact) <= 4
    scale, words, _ = oracle_w4(orc, fast)
    gw, gs = ops.absmax_quantize(w.cuda(), qtype=ops.QINT, bits=4, col_group=128, codec="pack32", hadamard_n=128,
                                 signs=sg.cuda(), precision=precision)
    assert_bit_equal(gs.cpu(), scale, "scales from our rotated tensor")
    assert_bit_equal(gw.cpu(), words, "packed words from our rotated tensor")


def test_tensor_core_path_batch_and_limits(ops, orc):
    """The tcgen05 path over a table of tensors (one tensor map spanning all of them) equals its own single-tensor
    calls; shapes that are not whole 128 x 128 tiles are refused; the device status word stays clear."""
    from compressed_tensors_b200.parallel import ShardCodec

    sg = signs128(6).cuda()
    ws = [weights(r, c, seed=40 + i).cuda() for i, (r, c) in enumerate([(128, 128), (1024, 4096), (32, 512), (512, 14336)])]
    codec = ShardCodec(ws, signs=sg, precision=ops.ROT_TENSOR)
    codec.compress(), codec.decompress()
    torch.cuda.synchronize()
    assert int(codec.status.item()) == 0
    for i, w in enumerate(ws):
        gw, gs = ops.absmax_quantize(w, qtype=ops.QINT, bits=4, col_group=128, codec="pack32", hadamard_n=128, signs=sg,
                                     precision=ops.ROT_TENSOR)
        assert_bit_equal(codec.packed[i].cpu(), gw.cpu(), f"words {i}")
        assert_bit_equal(codec.scales[i].cpu(), gs.cpu(), f"scales {i}")
    with pytest.raises(NotImplementedError):
        ops.hadamard(weights(3, 128).cuda(), 128, signs=sg, precision=ops.ROT_TENSOR)


def test_fp8_channel_and_token_match_oracle(ops, orc):
    w = weights(512, 4096, seed=3)
    mn, mx = orc.minmax(w, 1, 4096)
    scale, zp = orc.calculate_qparams(mn, mx, qtype=orc.QFLOAT, bits=8, symmetric=True)
    kw = dict(qtype=orc.QFLOAT, bits=8, col_group=4096, row_group=1, scale_row_stride=1)
    q = orc.quantize(w, scale, zp, out_dtype=torch.float8_e4m3fn, **kw)
    deq = orc.dequantize(q, scale, zp, out_dtype=torch.bfloat16, **kw)
    gq, gs = ops.absmax_quantize(w.cuda(), qtype=ops.QFLOAT, bits=8, col_group=4096, codec="dtype", out_dtype=torch.float8_e4m3fn)
    assert_bit_equal(gs.cpu(), scale.reshape(gs.shape), "per-channel scales")
    assert_bit_equal(gq.cpu(), q, "e4m3 codes")
    assert_bit_equal(ops.dequantize(gq, gs, None, out_dtype=torch.bfloat16, **kw).cpu().view(torch.int16),
                     orc.dequantize(q, scale, None, out_dtype=torch.bfloat16, **kw).view(torch.int16), "dequantized")
    # activations with outlier channels, fp32 scales
    g = torch.Generator().manual_seed(4)
    x = torch.randn(1, 256, 4096, generator=g)
    x[..., torch.randperm(4096, generator=g)[:41]] *= 20
    x = x.to(torch.bfloat16)
    mn, mx = orc.minmax(x.float(), 1, 4096)
    s32, z32 = orc.calculate_qparams(mn, mx, qtype=orc.QFLOAT, bits=8, symmetric=True)
    q = orc.quantize(x, s32, z32, out_dtype=torch.float8_e4m3fn, **kw)
    assert_bit_equal(ops.quantize(x.cuda(), s32.cuda(), z32.cuda(), out_dtype=torch.float8_e4m3fn, **kw).cpu(), q, "fp32-scale codes")
    assert_bit_equal(ops.dequantize(q.cuda(), s32.cuda(), z32.cuda(), out_dtype=torch.float32, **kw).cpu(),
                     orc.dequantize(q, s32, z32, out_dtype=torch.float32, **kw), "fp32-scale dequantized")
    assert deq.dtype == torch.bfloat16


def test_nvfp4_matches_oracle(ops, orc):
    w = weights(512, 4096, seed=6)
    mn, mx = orc.minmax(w, 512, 4096)
    gs = orc.generate_gparam(mn, mx)
    gmn, gmx = orc.minmax(w, 1, 16)
    scale, _ = orc.calculate_qparams(gmn, gmx, qtype=orc.QFLOAT, bits=4, symmetric=True, global_scale=gs)
    kw = dict(qtype=orc.QFLOAT, bits=4, col_group=16, row_group=1, scale_row_stride=256, global_scale=gs)
    packed = orc.pack_fp4(orc.quantize(w, scale, None, out_dtype=torch.bfloat16, **kw))
    deq = orc.dequantize(orc.unpack_fp4(packed, 512, 4096), scale, None, out_dtype=torch.bfloat16, **kw)
    dmn, dmx = ops.minmax(w.cuda(), 512, 4096)
    dgs = ops.generate_gparam(dmn, dmx)
    assert_bit_equal(dgs.cpu(), gs, "global scale")
    gp, gsc = ops.absmax_quantize(w.cuda(), qtype=ops.QFLOAT, bits=4, col_group=16, codec="fp4x2", global_scale=dgs)
    assert_bit_equal(gsc.cpu(), scale, "e4m3 group scales")
    assert_bit_equal(gp.cpu(), packed, "packed e2m1 bytes")
    kwd = dict(kw, global_scale=dgs)
    assert_bit_equal(ops.dequantize(gp, gsc, None, out_dtype=torch.bfloat16, codec="fp4x2", **kwd).cpu(), deq, "dequantized")


def test_sparse_codecs_match_oracle(ops, orc):
    g = torch.Generator().manual_seed(7)
    w = weights(256, 2048, seed=7)
    w[torch.rand(256, 2048, generator=g) < 0.5] = 0
    values, bitmask, row_offsets = orc.bitmask_compress(w)
    gv, gb, gr = ops.bitmask_compress(w.cuda())
    assert_bit_equal(gv.cpu(), values), assert_bit_equal(gb.cpu(), bitmask), assert_bit_equal(gr.cpu(), row_offsets)
    assert_bit_equal(ops.bitmask_decompress(gv, gb, w.shape).cpu(), orc.bitmask_decompress(values, bitmask, w.shape))
    for t in (weights(256, 2048, seed=8), weights(256, 2048, seed=9).to(torch.float8_e4m3fn)):
        mask = orc.sparse24_mask(t)
        pruned = torch.where(mask, t.float(), torch.zeros(())).to(t.dtype)
        v, b = orc.sparse24_compress(pruned)
        dv, db = ops.sparse24_compress(pruned.cuda())
        assert_bit_equal(dv.cpu(), v), assert_bit_equal(db.cpu(), b)
        assert_bit_equal(ops.sparse24_mask(t.cuda()).cpu(), mask, "keep mask on unpruned values")
        assert_bit_equal(ops.bitmask_decompress(dv, db, t.shape).cpu(), orc.bitmask_decompress(v, b, t.shape))
    # the 2:4 decompress entry: scan-free on a regular mask, generic kernels take over on an irregular one
    t = weights(64, 512, seed=12)
    v, b = ops.sparse24_compress(t.cuda())
    assert_bit_equal(ops.sparse24_decompress(v, b, t.shape).cpu(), ops.bitmask_decompress(v, b, t.shape).cpu(), "regular 2:4 mask")
    vals, bm, _ = ops.bitmask_compress(w.cuda())  # unstructured: not two-per-four
    assert_bit_equal(ops.sparse24_decompress(vals, bm, w.shape).cpu(), orc.bitmask_decompress(values, bitmask, w.shape), "irregular mask")
    # ops run twice give identical bits (no race in the compaction)
    gv2, gb2, gr2 = ops.bitmask_compress(w.cuda())
    assert_bit_equal(gv2.cpu(), gv.cpu()), assert_bit_equal(gr2.cpu(), gr.cpu())


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32, torch.int8, torch.float8_e4m3fn])
@pytest.mark.parametrize("shape", [(1, 8), (3, 8), (37, 24), (129, 1000), (5, 13), (700, 4096)])
@pytest.mark.parametrize("density", [0.0, 0.03, 0.5, 1.0])
@pytest.mark.parametrize("two_kernels", [False, True])
def test_bitmask_codec_shapes_dtypes_densities(ops, orc, dtype, shape, density, two_kernels, request):
    """ragged tile counts, every element size, empty / sparse / dense tensors, and a row length that is not a
    multiple of 8 (the row-by-row kernels), all bit-exact against the oracle; once through the single-pass compress
    kernel and once through the count + compaction pair"""
    from compressed_tensors_b200 import _lib as L

    L.lib().ctb_bitmask_force_two_kernels(L.i32(1 if two_kernels else 0))
    request.addfinalizer(lambda: L.lib().ctb_bitmask_force_two_kernels(L.i32(1)))
    g = torch.Generator().manual_seed(hash((shape, density)) % 1000)
    if dtype == torch.int8:
        w = torch.randint(1, 128, shape, generator=g).float()
    else:
        w = torch.randn(shape, generator=g) + 3.0  # no zeros before the mask is applied
    w[torch.rand(shape, generator=g) >= density] = 0
    w = w.to(dtype)
    values, bitmask, row_offsets = orc.bitmask_compress(w)
    gv, gb, gr = ops.bitmask_compress(w.cuda())
    assert_bit_equal(gb.cpu(), bitmask, "bitmask"), assert_bit_equal(gr.cpu(), row_offsets, "row offsets")
    assert_bit_equal(gv.cpu(), values, "values")
    assert_bit_equal(ops.bitmask_decompress(gv, gb, w.shape).cpu(), orc.bitmask_decompress(values, bitmask, w.shape), "dense")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32, torch.int8, torch.float8_e4m3fn])
@pytest.mark.parametrize("shape", [(1, 8), (3, 8), (37, 24), (129, 1000), (700, 4096)])
def test_sparse24_codec_shapes_dtypes(ops, orc, dtype, shape):
    """odd unit counts (the half-filled last thread) and every element size through the fused 2:4 kernels; small
    integer magnitudes make ties the common case"""
    g = torch.Generator().manual_seed(sum(shape))
    t = torch.randint(-3, 4, shape, generator=g)
    t = t.to(torch.int8) if dtype == torch.int8 else (t * 0.5).to(dtype)
    v, b = orc.sparse24_compress(t)
    dv, db = ops.sparse24_compress(t.cuda())
    assert_bit_equal(db.cpu(), b, "bitmask"), assert_bit_equal(dv.cpu(), v, "values")
    assert_bit_equal(ops.sparse24_decompress(dv, db, t.shape).cpu(), orc.bitmask_decompress(v, b, t.shape), "dense")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32, torch.int8, torch.float8_e4m3fn])
@pytest.mark.parametrize("shape", [(1, 4), (3, 4), (5, 12), (37, 24), (129, 1000), (700, 4096)])
def test_sparse24_mask_shapes_dtypes(ops, orc, dtype, shape):
    """get_24_bytemasks: sizes that are not a whole number of 16-byte chunks (scalar tail behind the SIMD kernel),
    every element size, small integer magnitudes so that ties are the common case"""
    g = torch.Generator().manual_seed(sum(shape) + 1)
    t = torch.randint(-3, 4, shape, generator=g)
    t = t.to(torch.int8) if dtype == torch.int8 else (t * 0.5).to(dtype)
    assert_bit_equal(ops.sparse24_mask(t.cuda()).cpu(), orc.sparse24_mask(t), "keep mask")


@pytest.mark.parametrize("bits", [4, 8])
def test_marlin24_steps_match_oracle(ops, orc, bits):
    """the Marlin-24 kernels against the oracle on a weight-sized tensor with every non-zero pattern of a run"""
    g = torch.Generator().manual_seed(24 + bits)
    n, k = 512, 2048
    half = (1 << bits) // 2
    q = torch.randint(-half, half, (n, k), generator=g, dtype=torch.int8)
    q[torch.rand(n, k, generator=g) < 0.55] = 0  # runs with 0..4 non-zeros: every branch of the index selection
    sparse, meta = orc.cutlass24_compress(q)
    gs, gm = ops.cutlass24_compress(q.cuda())
    assert_bit_equal(gs.cpu(), sparse, "2:4 values"), assert_bit_equal(gm.cpu(), meta, "reordered meta")
    assert_bit_equal(ops.marlin24_pack_weight(gs, bits).cpu(), orc.marlin24_pack_weight(sparse, bits), "packed weight")
    scale = torch.rand(n, k // 128, generator=g).to(torch.float16)
    for grouped in (False, True):
        assert_bit_equal(ops.marlin24_pack_scales(scale.cuda(), grouped).cpu(), orc.marlin24_pack_scales(scale, grouped), "scales")


@pytest.mark.parametrize("shape", [(14336, 4096), (4096, 14336), (1024, 4096)])
def test_full_size_round_trip_properties(ops, shape):
    """At the benchmark's tensor sizes: compress -> decompress -> compress is a fixed point (same words, same
    scales), the dequantized tensor equals fake-quantize of the rotated tensor, and the reconstruction error is
    bounded by half a quantization step per element."""
    g = torch.Generator(device="cuda").manual_seed(11)
    w = (torch.randn(shape, generator=g, device="cuda") * 0.02).to(torch.bfloat16)
    sg = signs128(3).cuda()
    words, scale = ops.absmax_quantize(w, qtype=ops.QINT, bits=4, col_group=128, codec="pack32", hadamard_n=128, signs=sg,
                                       precision=torch.float64)
    kw = dict(qtype=ops.QINT, bits=4, col_group=128, scale_row_stride=shape[1] // 128)
    deq = ops.dequantize(words, scale, None, out_dtype=torch.bfloat16, codec="pack32", cols=shape[1], **kw)
    rot = ops.hadamard(w, 128, signs=sg, precision=torch.float64)
    fake = ops.fake_quantize(rot, scale, None, out_dtype=torch.bfloat16, **kw)
    # equal as numbers: an int4 code has no -0, fake_quantize keeps the sign of a zero quotient (as in the reference)
    assert torch.equal(deq, fake), "decompress == fake_quantize(rotated)"
    again = ops.quantize(deq, scale, None, codec="pack32", **kw)
    assert torch.equal(again, words), "re-quantizing the dequantized tensor with the same scales is the identity"
    step = scale.float().repeat_interleave(128, dim=1)
    assert bool(((deq.float() - rot.float()).abs() <= 0.56 * step + 1e-9).all())
    # rotation is orthogonal: the inverse rotation restores the weights to bf16 accuracy
    back = ops.hadamard(rot, 128, signs=sg, inverse=True, precision=torch.float64)
    rel = (back.float() - w.float()).norm() / w.float().norm()
    assert float(rel) < 5e-3
    # words checksum is reproducible run to run
    words2, _ = ops.absmax_quantize(w, qtype=ops.QINT, bits=4, col_group=128, codec="pack32", hadamard_n=128, signs=sg,
                                    precision=torch.float64)
    assert int(words.to(torch.int64).sum()) == int(words2.to(torch.int64).sum())


@pytest.mark.parametrize("shape", [(14336, 4096), (4096, 11008)])
def test_full_size_sparse_codec_properties(ops, shape):
    """At the benchmark's tensor sizes, through properties that need no CPU pass over the tensor: bitmask and 2:4
    round trips restore the input bit for bit, counts agree with the bitmask, row offsets are the running counts,
    the 2:4 mask keeps exactly two per run and never a smaller magnitude over a larger one."""
    g = torch.Generator(device="cuda").manual_seed(13)
    w = (torch.randn(shape, generator=g, device="cuda") * 0.02).to(torch.bfloat16)
    w[torch.rand(shape, generator=g, device="cuda") < 0.5] = 0
    values, bitmask, row_offsets = ops.bitmask_compress(w)
    nz = w != 0
    assert values.numel() == int(nz.sum())
    assert torch.equal(ops.unpack_bitmasks(bitmask, list(shape)), nz)
    counts = nz.sum(dim=1)
    assert torch.equal(row_offsets, torch.cumsum(counts, 0) - counts)
    assert torch.equal(values, w[nz]), "kept values in row-major order"
    assert_bit_equal(ops.bitmask_decompress(values, bitmask, shape).cpu(), torch.where(nz, w, torch.zeros((), dtype=w.dtype, device="cuda")).cpu())
    # 2:4
    d = (torch.randn(shape, generator=g, device="cuda") * 0.02).to(torch.bfloat16)
    keep = ops.sparse24_mask(d)
    assert bool((keep.view(-1, 4).sum(dim=1) == 2).all())
    mag = d.abs().float().view(-1, 4)
    kept_min = torch.where(keep.view(-1, 4), mag, torch.full_like(mag, float("inf"))).amin(dim=1)
    drop_max = torch.where(keep.view(-1, 4), torch.full_like(mag, -1.0), mag).amax(dim=1)
    assert bool((kept_min >= drop_max).all()), "no dropped element is larger than a kept one"
    pruned = torch.where(keep, d, torch.zeros((), dtype=d.dtype, device="cuda"))
    v24, b24 = ops.sparse24_compress(pruned)
    assert torch.equal(ops.unpack_bitmasks(b24, list(shape)), ops.sparse24_mask(pruned)), "bitmask == mask of the pruned tensor"
    assert torch.equal(v24.flatten(), pruned[ops.unpack_bitmasks(b24, list(shape))])
    assert torch.equal(ops.sparse24_decompress(v24, b24, shape), pruned)


def test_full_size_fp8_and_nvfp4_properties(ops):
    """FP8 per-token activations (8192 x 4096) and NVFP4 weights (14336 x 4096): fused calibrate+quantize equals the
    separate calls, dequantize(quantize) is a fixed point of quantize, and the error stays inside half a step."""
    g = torch.Generator(device="cuda").manual_seed(17)
    x = torch.randn(8192, 4096, generator=g, device="cuda").to(torch.bfloat16)
    kw8 = dict(qtype=ops.QFLOAT, bits=8, col_group=4096)
    q, s = ops.absmax_quantize(x, codec="dtype", out_dtype=torch.float8_e4m3fn, **kw8)
    mn, mx = ops.minmax(x, 1, 4096)
    amax = torch.maximum(mn.abs(), mx.abs()).float()
    assert torch.equal(s.float().flatten(), torch.clamp((amax / 448.0).to(torch.bfloat16).float(), min=torch.finfo(torch.float32).eps).flatten())
    assert_bit_equal(ops.quantize(x, s, None, out_dtype=torch.float8_e4m3fn, scale_row_stride=1, **kw8).cpu(), q.cpu(), "fused == separate")
    deq = ops.dequantize(q, s, None, scale_row_stride=1, out_dtype=torch.bfloat16, **kw8)
    assert bool(((deq.float() - x.float()).abs() <= 0.0725 * x.float().abs() + 2.0 ** -9 * s.float()).all()), "e4m3 relative step"
    w = (torch.randn(14336, 4096, generator=g, device="cuda") * 0.02).to(torch.bfloat16)
    mn, mx = ops.minmax(w, 14336, 4096)
    gs = ops.generate_gparam(mn, mx)
    kw4 = dict(qtype=ops.QFLOAT, bits=4, col_group=16)
    p, sc = ops.absmax_quantize(w, codec="fp4x2", global_scale=gs, **kw4)
    assert_bit_equal(ops.quantize(w, sc, None, codec="fp4x2", global_scale=gs, scale_row_stride=256, **kw4).cpu(), p.cpu(), "fused == separate")
    deq = ops.dequantize(p, sc, None, scale_row_stride=256, out_dtype=torch.bfloat16, codec="fp4x2", global_scale=gs, **kw4)
    again = ops.quantize(deq, sc, None, codec="fp4x2", global_scale=gs, scale_row_stride=256, **kw4)
    # the codes agree except that a negative value that rounded to zero keeps its sign bit (0x8) the first time only
    deq2 = ops.dequantize(again, sc, None, scale_row_stride=256, out_dtype=torch.bfloat16, codec="fp4x2", global_scale=gs, **kw4)
    assert torch.equal(deq2, deq), "re-quantizing the dequantized tensor with the same scales restores the same values"
    assert bool((((again ^ p) & 0x77) == 0).all()), "magnitude bits of every code are a fixed point"
    eff = (sc.float() / gs).repeat_interleave(16, dim=1)
    assert bool(((deq.float() - w.float()).abs() <= 1.01 * eff).all()), "inside one e2m1 step of the largest magnitudes"


@pytest.mark.parametrize("n", [32, 64, 128, 256, 512])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_weight_output_rotation_sizes(ops, orc, n, dtype):
    """rows-direction Hadamard (weight_output): every built size, both 16-bit dtypes, forward and inverse, with random
    signs, on shapes whose column count is not a whole tile; float64 mode bit-exact against the oracle, float32 mode
    within one step of the tensor dtype"""
    g = torch.Generator().manual_seed(n)
    signs = (torch.randint(0, 2, (n,), generator=g) * 2 - 1).to(torch.int8)
    for rows, cols in ((n, 36), (2 * n, 200), (n, 4096)):
        w = (torch.randn(rows, cols, generator=g) * 0.05).to(dtype)
        for inverse in (False, True):
            want = orc.hadamard(w, n, signs=signs, inverse=inverse, side=1)
            got = ops.hadamard(w.cuda(), n, signs=signs.cuda(), inverse=inverse, side=1, precision=torch.float64).cpu()
            assert_bit_equal(got, want, f"n={n} {rows}x{cols} inverse={inverse}")
            fast = ops.hadamard(w.cuda(), n, signs=signs.cuda(), inverse=inverse, side=1, precision=torch.float32).cpu()
            err = (fast.float() - want.float()).abs()
            step = want.float().abs() * (2.0 ** -7 if dtype == torch.bfloat16 else 2.0 ** -10) + 1e-6
            assert bool((err <= step).all()), f"n={n} float32 mode"


def test_vector_pack_kernels_match_oracle(ops, orc):
    """pack_to_int32 / unpack_from_int32 / pack_bitmasks / unpack_bitmasks on shapes that take the 16-bytes-per-thread
    kernels, against the oracle, including codes outside the field range (whose reference result spills into the
    neighbouring fields) and mask bytes other than 0 / 1"""
    g = torch.Generator().manual_seed(3)
    for bits in (4, 8):
        half = 1 << (bits - 1)
        q = torch.randint(-half, half, (96, 1024), generator=g, dtype=torch.int8)
        if bits == 4:
            q[5, 17], q[5, 18], q[40, 0], q[95, 1023] = 100, -100, 127, -128  # out of range for 4 bits
        want = orc.pack_int32(q, bits)
        got = ops.pack_int32(q.cuda(), bits)
        assert_bit_equal(got.cpu(), want, f"pack {bits}")
        inside = q.clamp(-half, half - 1)
        words = orc.pack_int32(inside, bits)
        assert_bit_equal(ops.unpack_int32(words.cuda(), bits, (96, 1024)).cpu(), inside, f"unpack {bits}")
        assert_bit_equal(ops.unpack_int32(words.cuda(), bits, (96, 1024)).cpu(), orc.unpack_int32(words, bits, (96, 1024)), f"unpack vs oracle {bits}")
    m = torch.randint(0, 3, (64, 2048), generator=g, dtype=torch.uint8) * 127  # 0, 127, 254: any non-zero byte is "set"
    m[3] = 0
    m[7] = 255
    want = orc.pack_bitmasks(m.bool())
    assert_bit_equal(ops.pack_bitmasks(m.bool().cuda()).cpu(), want, "pack_bitmasks")
    assert_bit_equal(ops.unpack_bitmasks(want.cuda(), [64, 2048]).cpu(), m.bool(), "unpack_bitmasks")


def test_whole_shard_batch_equals_per_tensor(ops):
    """One grid over a list of tensors (ragged sizes, a tensor smaller than one warp of blocks) gives exactly
    the per-tensor results, in both rotation precisions, and decompress restores the same values."""
    from compressed_tensors_b200.parallel import ShardCodec

    shapes = [(3, 128), (64, 256), (1024, 4096), (17, 384), (256, 14336), (1, 128)]
    ws = [weights(r, c, seed=20 + i).cuda() for i, (r, c) in enumerate(shapes)]
    sg = signs128(5).cuda()
    for precision in (torch.float64, torch.float32):
        batched = ShardCodec(ws, signs=sg, precision=precision, batch=True)
        single = ShardCodec(ws, signs=sg, precision=precision, batch=False)
        assert batched.batched and not single.batched
        batched.compress(), single.compress()
        batched.decompress(), single.decompress()
        for i in range(len(ws)):
            assert_bit_equal(batched.scales[i].cpu(), single.scales[i].cpu(), f"scales of tensor {i}")
            assert_bit_equal(batched.packed[i].cpu(), single.packed[i].cpu(), f"words of tensor {i}")
            assert_bit_equal(batched.restored[i].cpu(), single.restored[i].cpu(), f"restored tensor {i}")
    # and through CUDA graphs
    exact = ShardCodec(ws, signs=sg, precision=torch.float64, batch=False)
    exact.compress()
    graphed = ShardCodec(ws, signs=sg, precision=torch.float64, batch=True, use_graphs=True)
    for _ in range(2):
        graphed.compress(), graphed.decompress()
    torch.cuda.synchronize()
    for i in range(len(ws)):
        assert_bit_equal(graphed.packed[i].cpu(), exact.packed[i].cpu(), "graph replay")


def _same_bits_or_both_nan(a, b, what):
    assert a.dtype == b.dtype and tuple(a.shape) == tuple(b.shape), what
    if a.dtype == torch.float8_e4m3fn:
        ba, bb = a.view(torch.uint8), b.view(torch.uint8)
        ok = ba == bb  # e4m3 NaN codes carry the input's sign: compared as bits
    else:
        from tests.helpers import bits_of
        ok = (bits_of(a) == bits_of(b)) | (a.float().isnan() & b.float().isnan())
    bad = (~ok).flatten().nonzero().flatten()
    assert bad.numel() == 0, f"{what}: {bad.numel()} differ; first at {int(bad[0])}: {a.flatten()[int(bad[0])].item()!r} vs {b.flatten()[int(bad[0])].item()!r}"


def test_bf16_quantize_and_fake_quantize_kernels_match_oracle(ops, orc):
    """quantize (packed int4 / int8 / e4m3 codes) and fake_quantize of a bf16 tensor with bf16 scales (the path that
    stays in packed bf16x2 arithmetic) and with fp32 scales (fp32 quotients), against the oracle: rounding ties, both clamp ends, -0.0 results, infinities,
    NaNs where the reference defines the result, zero points, scales outside the fast range (tiny, huge, zero,
    infinite, NaN), GROUP / CHANNEL / BLOCK layouts with power-of-two and other group sizes"""
    g = torch.Generator().manual_seed(77)
    rows, cols = 192, 768
    base = torch.randn(rows, cols, generator=g) * 0.02
    layouts = [(1, 128, "group128"), (1, 96, "group96"), (1, cols, "channel"), (64, 96, "block64x96"), (rows, cols, "tensor")]
    for rg, cg, name in layouts:
        srs = cols // cg
        for qtype, bits in ((orc.QINT, 4), (orc.QINT, 8), (orc.QINT, 6), (orc.QFLOAT, 8)):
            is_int = qtype == orc.QINT
            x = base.clone()
            mn, mx = orc.minmax(x.to(torch.bfloat16), rg, cg)
            scale, _ = orc.calculate_qparams(mn, mx, qtype=qtype, bits=bits, symmetric=True)
            sf = scale.float().reshape(rows // rg, srs)
            # plant, per row-group 0 / qparam 0..: ties, clamp ends, signed zeros, infinities
            half = (1 << (bits - 1)) if is_int else 448
            s00 = float(sf[0, 0])
            ks = torch.arange(-half - 2, half + 2, dtype=torch.float32)
            plant = torch.cat([(ks + 0.5) * s00, ks * s00, torch.tensor([-0.0, 0.0, -1e-9, 1e-9, float("inf"), float("-inf")])])
            n_plant = min(plant.numel(), cg)
            x[0, :n_plant] = plant[:n_plant]
            special = [1e-38, 2.0 ** 100]        # outside the fast range: recomputed by the float path
            if not is_int:
                special += [0.0, float("inf"), float("nan")]
            flat = scale.reshape(-1).clone()
            for i, v in enumerate(special):
                if flat.numel() > 2 + i:
                    flat[2 + i] = v
            scale = flat.reshape(scale.shape)
            xb = x.to(torch.bfloat16)
            if not is_int:
                xb[1, 5], xb[1, 6] = float("nan"), -float("nan")
            zps = [None, torch.zeros(scale.shape, dtype=torch.int8 if is_int else torch.float8_e4m3fn)]
            if is_int:
                zps.append(torch.randint(-half // 2, half // 2, scale.shape, generator=g, dtype=torch.int8))
            else:
                nz = torch.zeros(scale.shape, dtype=torch.float32)
                nz.reshape(-1)[0] = 2.0  # an fp8 zero point other than zero: float path
                zps.append(nz.to(torch.float8_e4m3fn))
            # the same scales in fp32 (compute dtype fp32), exact and perturbed so that the quotients are not bf16-friendly
            jitter = 1.0 + 1e-3 * torch.rand(scale.shape, generator=g)
            variants = [(scale, "bf16 scale"), (scale.float(), "fp32 scale"), (scale.float() * jitter, "fp32 scale, perturbed")]
            for (scale, stag), (zi, zp) in itertools.product(variants, enumerate(zps)):
                kw = dict(qtype=qtype, bits=bits, col_group=cg, row_group=rg, scale_row_stride=srs)
                dz = None if zp is None else zp.cuda()
                what = f"{name} bits={bits} {'int' if is_int else 'fp8'} zp#{zi} {stag}"
                code_dt = torch.int8 if is_int else torch.float8_e4m3fn
                want = orc.quantize(xb, scale, zp, out_dtype=code_dt, **kw)
                got = ops.quantize(xb.cuda(), scale.cuda(), dz, out_dtype=code_dt, **kw)
                _same_bits_or_both_nan(got.cpu(), want, "quantize " + what)
                if is_int and bits in (4, 8) and rg == 1:
                    words = ops.quantize(xb.cuda(), scale.cuda(), dz, codec="pack32", **kw)
                    assert_bit_equal(words.cpu(), orc.pack_int32(want, bits), "pack32 " + what)
                xf = xb.clone()
                xf[2, 3] = float("nan")  # fake quantize: a NaN stays a NaN
                wantf = orc.fake_quantize(xf, scale, zp, out_dtype=torch.bfloat16, **kw)
                gotf = ops.fake_quantize(xf.cuda(), scale.cuda(), dz, out_dtype=torch.bfloat16, **kw)
                _same_bits_or_both_nan(gotf.cpu(), wantf, "fake_quantize " + what)


def test_activation_ordered_groups_match_oracle(ops, orc):
    """g_idx (a group number per column, forward.py:300-352) through the 8-wide kernels: int8 codes, packed words,
    dequantize from both, fake quantize; symmetric and asymmetric; bf16 and f16"""
    g = torch.Generator().manual_seed(31)
    rows, cols, group = 96, 512, 64
    perm = torch.randperm(cols, generator=g)
    g_idx = torch.empty(cols, dtype=torch.int32)
    g_idx[perm] = (torch.arange(cols) // group).to(torch.int32)
    for dt in (torch.bfloat16, torch.float16):
        x = (torch.randn(rows, cols, generator=g) * 0.05 + 0.01).to(dt)
        xs = x.index_select(-1, torch.argsort(g_idx))
        mn, mx = orc.minmax(xs, 1, group)
        for sym in (True, False):
            scale, zp = orc.calculate_qparams(mn, mx, qtype=orc.QINT, bits=4, symmetric=sym)
            if dt == torch.bfloat16:
                scale[3, 1], scale[5, 0] = 1e-38, 2.0 ** 100  # rows with a scale outside the fast range take the float path
            kw = dict(qtype=orc.QINT, bits=4, col_group=group, row_group=1, scale_row_stride=cols // group)
            want = orc.quantize(x, scale, zp, out_dtype=torch.int8, g_idx=g_idx, **kw)
            dz, dg = zp.cuda(), g_idx.cuda()
            got = ops.quantize(x.cuda(), scale.cuda(), dz, out_dtype=torch.int8, g_idx=dg, **kw)
            assert_bit_equal(got.cpu(), want, f"codes {dt} sym={sym}")
            words = ops.quantize(x.cuda(), scale.cuda(), dz, codec="pack32", g_idx=dg, **kw)
            assert_bit_equal(words.cpu(), orc.pack_int32(want, 4), f"words {dt} sym={sym}")
            wantd = orc.dequantize(want, scale, zp, out_dtype=dt, g_idx=g_idx, **kw)
            assert_bit_equal(ops.dequantize(got, scale.cuda(), dz, out_dtype=dt, g_idx=dg, **kw).cpu(), wantd, f"dequant {dt} sym={sym}")
            assert_bit_equal(ops.dequantize(words, scale.cuda(), dz, out_dtype=dt, codec="pack32", cols=cols, g_idx=dg, **kw).cpu(), wantd,
                             f"dequant from words {dt} sym={sym}")
            wantf = orc.fake_quantize(x, scale, zp, out_dtype=dt, g_idx=g_idx, **kw)
            assert_bit_equal(ops.fake_quantize(x.cuda(), scale.cuda(), dz, out_dtype=dt, g_idx=dg, **kw).cpu(), wantf, f"fake {dt} sym={sym}")


@pytest.mark.parametrize("n", [512, 1024, 4096, 8192])
def test_whole_dimension_rotation_sizes(ops, orc, n):
    """Hadamard transforms as wide as a hidden dimension, both weight sides, forward and inverse, random signs,
    bf16 and f16; float64 mode bit-exact against the oracle, float32 mode within one step of the tensor dtype.
    The weight_output shapes cover the wide-tile kernel (8, 4 or 2 columns per tile) and a column count it cannot
    tile (generic kernel)."""
    g = torch.Generator().manual_seed(n)
    signs = (torch.randint(0, 2, (n,), generator=g) * 2 - 1).to(torch.int8)
    for dtype in (torch.bfloat16, torch.float16):
        shapes = [(0, 3, n), (1, n, 8)] if n >= 4096 else [(0, 5, 2 * n), (1, 2 * n, 24), (1, n, 7)]
        for side, rows, cols in shapes:
            w = (torch.randn(rows, cols, generator=g) * 0.05).to(dtype)
            for inverse in (False, True):
                want = orc.hadamard(w, n, signs=signs, inverse=inverse, side=side)
                got = ops.hadamard(w.cuda(), n, signs=signs.cuda(), inverse=inverse, side=side, precision=torch.float64).cpu()
                assert_bit_equal(got, want, f"n={n} side={side} {rows}x{cols} inverse={inverse} {dtype}")
                fast = ops.hadamard(w.cuda(), n, signs=signs.cuda(), inverse=inverse, side=side, precision=torch.float32).cpu()
                err = (fast.float() - want.float()).abs()
                step = want.float().abs() * (2.0 ** -7 if dtype == torch.bfloat16 else 2.0 ** -10) + 1e-6
                assert bool((err <= step).all()), f"n={n} side={side} float32 mode"


def test_fused_dynamic_token_fake_quantize_equals_separate_kernels(ops, orc):
    """dynamic per-token fake quantization in one pass (min/max + qparams + fake_quantize of the row held in registers)
    against the three separate kernels and the oracle: int8 and fp8, outlier channels, an all-zero token, signed zeros"""
    g = torch.Generator().manual_seed(12)
    for cols in (256, 4096, 8192):
        x = torch.randn(96, cols, generator=g)
        x[:, torch.randperm(cols, generator=g)[: cols // 100 + 1]] *= 20
        x[5] = 0
        x[6, :8] = torch.tensor([-0.0, 0.0, -1e-30, 1e-30, 3.0, -3.0, 1e-3, -1e-3])
        x = x.to(torch.bfloat16)
        for qtype, zdt in ((orc.QINT, torch.int8), (orc.QFLOAT, torch.float8_e4m3fn)):
            mn, mx = orc.minmax(x, 1, cols)
            scale, zp = orc.calculate_qparams(mn, mx, qtype=qtype, bits=8, symmetric=True)
            kw = dict(qtype=qtype, bits=8, col_group=cols, row_group=1, scale_row_stride=1)
            want = orc.fake_quantize(x, scale, zp, out_dtype=torch.bfloat16, **kw)
            fused, fscale = ops.absmax_quantize(x.cuda(), qtype=qtype, bits=8, col_group=cols, codec="dtype", out_dtype=torch.bfloat16)
            assert_bit_equal(fscale.cpu().reshape(scale.shape), scale, f"scale {cols}")
            assert_bit_equal(fused.cpu(), want, f"fused fake quantize {cols} qtype={qtype}")
            dmn, dmx = ops.minmax(x.cuda(), 1, cols)
            dscale, dzp = ops.calculate_qparams(dmn, dmx, qtype=qtype, bits=8, symmetric=True)
            sep = ops.fake_quantize(x.cuda(), dscale, dzp, out_dtype=torch.bfloat16, **kw)
            assert_bit_equal(sep.cpu(), want, f"separate kernels {cols} qtype={qtype}")


def test_fused_dynamic_group_fake_quantize_matches_oracle(ops, orc):
    """dynamic per-group fake quantization in one pass (group-128 FP8 activations of the FP8_BLOCK preset, int8 and
    int4 groups) against the oracle's min/max -> qparams -> fake_quantize, and through forward_quantize"""
    from compressed_tensors_b200.quantization import QuantizationArgs, forward_quantize

    g = torch.Generator().manual_seed(13)
    x = torch.randn(64, 1024, generator=g)
    x[:, 17] *= 30
    x[3, :128] = 0
    x[4, :4] = torch.tensor([-0.0, 0.0, -1e-30, 1e-30])
    x = x.to(torch.bfloat16)
    for qtype, bits, group, tname in ((orc.QFLOAT, 8, 128, "float"), (orc.QINT, 8, 128, "int"), (orc.QINT, 4, 32, "int"), (orc.QINT, 8, 256, "int")):
        mn, mx = orc.minmax(x, 1, group)
        scale, zp = orc.calculate_qparams(mn, mx, qtype=qtype, bits=bits, symmetric=True)
        kw = dict(qtype=qtype, bits=bits, col_group=group, row_group=1, scale_row_stride=1024 // group)
        want = orc.fake_quantize(x, scale, zp, out_dtype=torch.bfloat16, **kw)
        fused, fscale = ops.absmax_quantize(x.cuda(), qtype=qtype, bits=bits, col_group=group, codec="dtype", out_dtype=torch.bfloat16)
        assert_bit_equal(fscale.cpu(), scale, f"scale g{group} {tname}{bits}")
        assert_bit_equal(fused.cpu(), want, f"fused g{group} {tname}{bits}")
        args = QuantizationArgs(num_bits=bits, type=tname, symmetric=True, strategy="group", group_size=group, dynamic=True)
        assert_bit_equal(forward_quantize(None, x.cuda().reshape(2, 32, 1024), "input", args).cpu().reshape(64, 1024), want, f"forward_quantize g{group}")


def test_tiny_and_odd_shapes_through_the_fast_kernels(ops, orc):
    """one row, one chunk, groups of 8 / 24 / 40 elements, blocks of 1 x 8 and 3 x 24, fewer chunks than a warp: the
    packed quantize / fake_quantize / dequantize kernels, the packed min / max kernels and the fused dynamic fake
    quantization against the oracle"""
    g = torch.Generator().manual_seed(99)
    shapes = [(1, 8, 1, 8), (1, 16, 1, 8), (3, 24, 1, 24), (3, 24, 3, 24), (5, 120, 1, 40), (5, 120, 5, 24), (2, 256, 1, 256), (7, 64, 7, 64),
              (33, 8, 1, 8), (1, 8200, 1, 8200)]
    for rows, cols, rg, cg in shapes:
        x = (torch.randn(rows, cols, generator=g) * 0.1).to(torch.bfloat16)
        mn, mx = orc.minmax(x, rg, cg)
        dmn, dmx = ops.minmax(x.cuda(), rg, cg)
        assert_bit_equal(dmn.cpu(), mn, f"min {rows}x{cols} tile {rg}x{cg}")
        assert_bit_equal(dmx.cpu(), mx, f"max {rows}x{cols} tile {rg}x{cg}")
        srs = cols // cg
        for qtype, bits, sym, code_dt in ((orc.QINT, 4, True, torch.int8), (orc.QINT, 8, False, torch.int8), (orc.QFLOAT, 8, True, torch.float8_e4m3fn)):
            scale, zp = orc.calculate_qparams(mn, mx, qtype=qtype, bits=bits, symmetric=sym)
            for sc in (scale, scale.float()):
                kw = dict(qtype=qtype, bits=bits, col_group=cg, row_group=rg, scale_row_stride=srs)
                what = f"{rows}x{cols} tile {rg}x{cg} bits={bits} {sc.dtype}"
                want = orc.quantize(x, sc, zp, out_dtype=code_dt, **kw)
                got = ops.quantize(x.cuda(), sc.cuda(), zp.cuda(), out_dtype=code_dt, **kw)
                assert_bit_equal(got.cpu(), want, "quantize " + what)
                assert_bit_equal(ops.fake_quantize(x.cuda(), sc.cuda(), zp.cuda(), out_dtype=torch.bfloat16, **kw).cpu(),
                                 orc.fake_quantize(x, sc, zp, out_dtype=torch.bfloat16, **kw), "fake " + what)
                assert_bit_equal(ops.dequantize(got, sc.cuda(), zp.cuda(), out_dtype=torch.bfloat16, **kw).cpu(),
                                 orc.dequantize(want, sc, zp, out_dtype=torch.bfloat16, **kw), "dequantize " + what)
        if rg == 1 and (cg == cols or cg & (cg - 1) == 0) and cols <= 8192:
            for qtype in (orc.QINT, orc.QFLOAT):
                scale, zp = orc.calculate_qparams(mn, mx, qtype=qtype, bits=8, symmetric=True)
                kw = dict(qtype=qtype, bits=8, col_group=cg, row_group=1, scale_row_stride=srs)
                fused, fs = ops.absmax_quantize(x.cuda(), qtype=qtype, bits=8, col_group=cg, codec="dtype", out_dtype=torch.bfloat16)
                assert_bit_equal(fs.cpu().reshape(scale.shape), scale, f"fused scale {rows}x{cols} g{cg}")
                assert_bit_equal(fused.cpu(), orc.fake_quantize(x, scale, zp, out_dtype=torch.bfloat16, **kw), f"fused fake {rows}x{cols} g{cg}")
