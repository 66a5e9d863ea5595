"""Bit-exact parity against the CPU oracle at the FULL tensor sizes of the benchmark configurations (the
oracle is C + OpenMP and finishes each of these in about a second), so that anything that depends on the
grid shape -- moving-window grids, tile-start tables, offsets beyond 2^31 bytes -- is compared and not
only checked for self-consistency.  Outputs are allocated between canary pages: a kernel that writes one
byte outside its output fails here even if the result is right."""
import os

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
    ref.set_threads(os.cpu_count() or 1)
    return ref


def weights(rows, cols, seed, std=0.02):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(rows, cols, generator=g) * std).to(torch.bfloat16)


def test_c1_w4a16_full(ops, orc, canary):
    """BASELINE config 1 at 4096 x 4096: scales, packed words, dequantized values."""
    w = weights(4096, 4096, 0)
    mn, mx = orc.minmax(w, 1, 128)
    scale, zp = orc.calculate_qparams(mn, mx, qtype=orc.QINT, bits=4, symmetric=True)
    kw = dict(qtype=orc.QINT, bits=4, col_group=128, row_group=1, scale_row_stride=32)
    words = orc.pack_int32(orc.quantize(w, scale, zp, out_dtype=torch.int8, **kw), 4)
    deq = orc.dequantize(orc.unpack_int32(words, 4, w.shape), scale, None, out_dtype=torch.bfloat16, **kw)
    with canary():
        gw, gs = ops.absmax_quantize(w.cuda(), qtype=ops.QINT, bits=4, col_group=128, codec="pack32")
        given = ops.quantize(w.cuda(), scale.cuda(), None, codec="pack32", **kw)
        gd = ops.dequantize(gw, gs, None, out_dtype=torch.bfloat16, codec="pack32", cols=4096, **kw)
    assert_bit_equal(gs.cpu(), scale, "scales")
    assert_bit_equal(gw.cpu(), words, "words (fused calibrate)")
    assert_bit_equal(given.cpu(), words, "words (given scales)")
    assert_bit_equal(gd.cpu(), deq, "dequantized")


def test_c2_fp8_full(ops, orc, canary):
    """BASELINE config 2: 4096 x 4096 weight with static per-channel scales, and [1, 8192, 4096] activations with 41
    outlier channels scaled x20, per-token dynamic scales; bf16 and fp32 scales."""
    w = weights(4096, 4096, 1)
    kw = dict(qtype=orc.QFLOAT, bits=8, col_group=4096, row_group=1, scale_row_stride=1)
    mn, mx = orc.minmax(w, 1, 4096)
    scale, zp = orc.calculate_qparams(mn, mx, qtype=orc.QFLOAT, bits=8, symmetric=True)
    q = orc.quantize(w, scale, zp, out_dtype=torch.float8_e4m3fn, **kw)
    with canary():
        gq, gs = ops.absmax_quantize(w.cuda(), qtype=ops.QFLOAT, bits=8, col_group=4096, codec="dtype", out_dtype=torch.float8_e4m3fn)
        gd = ops.dequantize(gq, gs, None, out_dtype=torch.bfloat16, **kw)
    assert_bit_equal(gs.cpu(), scale.reshape(gs.shape), "weight scales")
    assert_bit_equal(gq.cpu(), q, "weight codes")
    assert_bit_equal(gd.cpu(), orc.dequantize(q, scale, None, out_dtype=torch.bfloat16, **kw), "weight dequantized")
    g = torch.Generator().manual_seed(2)
    x = torch.randn(1, 8192, 4096, generator=g)
    x[..., torch.randperm(4096, generator=g)[:41]] *= 20
    x = x.to(torch.bfloat16)
    x2 = x.reshape(8192, 4096)
    mn, mx = orc.minmax(x2, 1, 4096)
    s16, z16 = orc.calculate_qparams(mn, mx, qtype=orc.QFLOAT, bits=8, symmetric=True)
    q16 = orc.quantize(x2, s16, z16, out_dtype=torch.float8_e4m3fn, **kw)
    with canary():
        gq, gs = ops.absmax_quantize(x.cuda(), qtype=ops.QFLOAT, bits=8, col_group=4096, codec="dtype", out_dtype=torch.float8_e4m3fn)
        gd = ops.dequantize(gq, gs, None, out_dtype=torch.bfloat16, **kw)
    assert_bit_equal(gs.cpu().reshape(-1), s16.reshape(-1), "token scales (bf16)")
    assert_bit_equal(gq.cpu().reshape(8192, 4096), q16, "token codes (bf16 scales)")
    assert_bit_equal(gd.cpu().reshape(8192, 4096), orc.dequantize(q16, s16, None, out_dtype=torch.bfloat16, **kw), "token dequantized")
    mn, mx = orc.minmax(x2.float(), 1, 4096)
    s32, z32 = orc.calculate_qparams(mn, mx, qtype=orc.QFLOAT, bits=8, symmetric=True)
    q32 = orc.quantize(x2, s32, z32, out_dtype=torch.float8_e4m3fn, **kw)
    with canary():
        gq = ops.quantize(x2.cuda(), s32.cuda(), z32.cuda(), out_dtype=torch.float8_e4m3fn, **kw)
        gd = ops.dequantize(gq, s32.cuda(), z32.cuda(), out_dtype=torch.float32, **kw)
    assert_bit_equal(gq.cpu(), q32, "token codes (fp32 scales)")
    assert_bit_equal(gd.cpu(), orc.dequantize(q32, s32, z32, out_dtype=torch.float32, **kw), "token dequantized (fp32)")


@pytest.mark.parametrize("shape", [(14336, 4096), (4096, 14336)])
def test_c3_nvfp4_full(ops, orc, canary, shape):
    """BASELINE config 3 at the gate/up and down shapes: global scale, e4m3 group scales, packed e2m1 bytes, dequantized."""
    rows, cols = shape
    w = weights(rows, cols, 3 + rows % 7)
    mn, mx = orc.minmax(w, rows, cols)
    gs = orc.generate_gparam(mn, mx)
    gmn, gmx = orc.minmax(w, 1, 16)
    scale, _ = orc.calculate_qparams(gmn, gmx, qtype=orc.QFLOAT, bits=4, symmetric=True, global_scale=gs)
    kw = dict(qtype=orc.QFLOAT, bits=4, col_group=16, row_group=1, scale_row_stride=cols // 16, global_scale=gs)
    packed = orc.pack_fp4(orc.quantize(w, scale, None, out_dtype=torch.bfloat16, **kw))
    deq = orc.dequantize(orc.unpack_fp4(packed, rows, cols), scale, None, out_dtype=torch.bfloat16, **kw)
    with canary():
        dmn, dmx = ops.minmax(w.cuda(), rows, cols)
        dgs = ops.generate_gparam(dmn, dmx)
        gp, gsc = ops.absmax_quantize(w.cuda(), qtype=ops.QFLOAT, bits=4, col_group=16, codec="fp4x2", global_scale=dgs)
        gd = ops.dequantize(gp, gsc, None, out_dtype=torch.bfloat16, codec="fp4x2", **dict(kw, global_scale=dgs))
    assert_bit_equal(dgs.cpu(), gs, "global scale")
    assert_bit_equal(gsc.cpu(), scale, "group scales")
    assert_bit_equal(gp.cpu(), packed, "packed bytes")
    assert_bit_equal(gd.cpu(), deq, "dequantized")


def test_c4a_sparse24_e4m3_full(ops, orc, canary):
    """BASELINE config 4a at 4096 x 11008: bf16 weights pruned 2:4, FP8 per-channel, 2:4 bitmask codec on the e4m3 tensor."""
    w = weights(4096, 11008, 4)
    mask = orc.sparse24_mask(w)
    pruned = torch.where(mask, w, torch.zeros((), dtype=w.dtype))
    kw = dict(qtype=orc.QFLOAT, bits=8, col_group=11008, row_group=1, scale_row_stride=1)
    mn, mx = orc.minmax(pruned, 1, 11008)
    scale, zp = orc.calculate_qparams(mn, mx, qtype=orc.QFLOAT, bits=8, symmetric=True)
    q = orc.quantize(pruned, scale, zp, out_dtype=torch.float8_e4m3fn, **kw)
    v, b = orc.sparse24_compress(q)
    with canary():
        gmask = ops.sparse24_mask(w.cuda())
        gq, _ = ops.absmax_quantize(pruned.cuda(), qtype=ops.QFLOAT, bits=8, col_group=11008, codec="dtype", out_dtype=torch.float8_e4m3fn)
        gv, gb = ops.sparse24_compress(gq)
        gd = ops.sparse24_decompress(gv, gb, q.shape)
    assert_bit_equal(gmask.cpu(), mask, "keep mask")
    assert_bit_equal(gq.cpu(), q, "e4m3 codes")
    assert_bit_equal(gb.cpu(), b, "bitmask")
    assert_bit_equal(gv.cpu(), v, "values")
    assert_bit_equal(gd.cpu(), orc.bitmask_decompress(v, b, q.shape), "decompressed")


def test_c4a_fused_quantize_sparse24_full(ops, orc, canary):
    """The same configuration through the one-pass kernel: bf16 weight + per-channel scale in, kept e4m3 values and
    bitmask out; with and without the (all-zero) zero point the calibrated module carries."""
    w = weights(4096, 11008, 4)
    pruned = torch.where(orc.sparse24_mask(w), w, torch.zeros((), dtype=w.dtype))
    pruned[7, :64] = -0.0  # signed zeros: the zero point decides whether their code keeps the sign, and the sign the rank
    kw = dict(qtype=orc.QFLOAT, bits=8, col_group=11008, row_group=1, scale_row_stride=1)
    mn, mx = orc.minmax(pruned, 1, 11008)
    scale, zp = orc.calculate_qparams(mn, mx, qtype=orc.QFLOAT, bits=8, symmetric=True)
    for z in (zp, None):
        v, b = orc.sparse24_compress(orc.quantize(pruned, scale, z, out_dtype=torch.float8_e4m3fn, **kw))
        with canary():
            gv, gb = ops.quantize_fp8_sparse24(pruned.cuda(), scale.cuda().reshape(-1), None if z is None else z.cuda().reshape(-1))
        assert_bit_equal(gb.cpu(), b, f"bitmask (zero point: {z is not None})")
        assert_bit_equal(gv.cpu(), v, f"values (zero point: {z is not None})")


def test_c4a_fused_sparse24_decompress_dequantize_full(ops, orc, canary):
    """The inverse of the one-pass compress at 4096 x 11008: kept e4m3 values + bitmask + per-channel scale in, bf16
    weight out, against the oracle's bitmask decompress followed by its dequantize; then a bitmask that is not
    two-per-four (the gated generic route) and a value buffer shorter than two per four (the ungated one)."""
    w = weights(4096, 11008, 4)
    pruned = torch.where(orc.sparse24_mask(w), w, torch.zeros((), dtype=w.dtype))
    kw = dict(qtype=orc.QFLOAT, bits=8, col_group=11008, row_group=1, scale_row_stride=1)
    mn, mx = orc.minmax(pruned, 1, 11008)
    scale, zp = orc.calculate_qparams(mn, mx, qtype=orc.QFLOAT, bits=8, symmetric=True)
    q = orc.quantize(pruned, scale, zp, out_dtype=torch.float8_e4m3fn, **kw)
    v, b = orc.sparse24_compress(q)
    want = orc.dequantize(orc.bitmask_decompress(v, b, q.shape), scale, None, out_dtype=torch.bfloat16, **kw)
    with canary():
        got = ops.sparse24_decompress_dequantize_fp8(v.cuda(), b.cuda(), scale.cuda().reshape(-1), q.shape)
    assert_bit_equal(got.cpu(), want, "fused decompress + dequantize")
    # irregular bitmasks on a smaller tensor: three-of-four and one-of-four runs, as the unstructured codec would write them
    g = torch.Generator().manual_seed(23)
    rows, cols = 257, 1032
    x = (torch.randn(rows, cols, generator=g) * 0.05).to(torch.bfloat16)
    x[torch.rand(rows, cols, generator=g) < 0.5] = 0
    kw = dict(qtype=orc.QFLOAT, bits=8, col_group=cols, row_group=1, scale_row_stride=1)
    mn, mx = orc.minmax(x, 1, cols)
    scale, zp = orc.calculate_qparams(mn, mx, qtype=orc.QFLOAT, bits=8, symmetric=True)
    q = orc.quantize(x, scale, None, out_dtype=torch.float8_e4m3fn, **kw)
    values, bitmask, _ = orc.bitmask_compress(q)
    want = orc.dequantize(orc.bitmask_decompress(values, bitmask, q.shape), scale, None, out_dtype=torch.bfloat16, **kw)
    x2 = x.clone()
    x2[::2] = 0  # every other row empty: far fewer values than two per run of four
    q2 = orc.quantize(x2, scale, None, out_dtype=torch.float8_e4m3fn, **kw)
    values2, bitmask2, _ = orc.bitmask_compress(q2)
    assert values2.numel() < rows * cols // 2 <= values.numel() + 4096
    want2 = orc.dequantize(orc.bitmask_decompress(values2, bitmask2, q.shape), scale, None, out_dtype=torch.bfloat16, **kw)
    room = torch.zeros(max(values.numel(), rows * cols // 2), dtype=torch.float8_e4m3fn)
    room[:values.numel()] = values  # a buffer with room for two per four, so the fast kernel runs first and opens the gate
    for name, vals, bitmask, want in (("short value buffer", values2, bitmask2, want2), ("full-size buffer, irregular bitmask", room, bitmask, want)):
        with canary():
            got = ops.sparse24_decompress_dequantize_fp8(vals.cuda(), bitmask.cuda(), scale.cuda().reshape(-1), q.shape)
        assert_bit_equal(got.cpu(), want, name)


def test_fused_quantize_sparse24_edge_cases(ops, orc, canary):
    """Dense (unpruned) rows so that ties and rank order matter, NaN / Inf / signed zeros, scales outside the range
    of the reciprocal shortcut, a zero point other than zero, a unit count that fills neither a warp nor a pair."""
    g = torch.Generator().manual_seed(17)
    rows, cols = 37, 104
    x = (torch.randn(rows, cols, generator=g) * 0.05).to(torch.bfloat16)
    x[0, :8] = torch.tensor([0.5, -0.5, float("inf"), -float("inf"), 0.0, -0.0, 1.0, -1.0]).to(torch.bfloat16)
    x.view(torch.int16)[0, 8:12] = torch.tensor([0x7FC0, -64, 0x7F81, -1], dtype=torch.int16)  # NaNs of both signs
    x[1] = x[1, 0]            # every run a four-way tie
    x[2, ::2] = -x[2, 1::2]   # magnitude ties between neighbours
    x[3] = 0
    x[4] = -0.0
    scale = (x.float().abs().nan_to_num(0, 0, 0).amax(dim=1) / 448).clamp_min(1e-6).to(torch.bfloat16)
    scale[5], scale[6], scale[8] = 2.0 ** -110, 2.0 ** 100, 2.0 ** -99
    x[5] = (torch.randn(cols, generator=g) * 2.0 ** -105).to(torch.bfloat16)
    x[6] = (torch.randn(cols, generator=g) * 2.0 ** 104).to(torch.bfloat16)
    kw = dict(qtype=orc.QFLOAT, bits=8, col_group=cols, row_group=1, scale_row_stride=1)
    zeros = torch.zeros(rows, dtype=torch.bfloat16)
    shifted = zeros.clone()
    shifted[9], shifted[10] = 3.0, -1.5
    for name, z in (("none", None), ("zeros", zeros), ("shifted", shifted), ("e4m3 zeros", zeros.to(torch.float8_e4m3fn))):
        want = orc.quantize(x, scale.reshape(-1, 1), None if z is None else z.reshape(-1, 1), out_dtype=torch.float8_e4m3fn, **kw)
        v, b = orc.sparse24_compress(want)
        with canary():
            gv, gb = ops.quantize_fp8_sparse24(x.cuda(), scale.cuda(), None if z is None else z.cuda())
            twice = ops.sparse24_compress(ops.quantize(x.cuda(), scale.cuda().reshape(-1, 1), None if z is None else z.cuda().reshape(-1, 1),
                                                       out_dtype=torch.float8_e4m3fn, **{**kw, "qtype": ops.QFLOAT}))
        assert_bit_equal(gb.cpu(), b, f"bitmask ({name})")
        assert_bit_equal(gv.cpu(), v, f"values ({name})")
        assert_bit_equal(gv.cpu(), twice[0].cpu(), f"values against the two-pass path ({name})")
        assert_bit_equal(gb.cpu(), twice[1].cpu(), f"bitmask against the two-pass path ({name})")
    assert ops.quantize_fp8_sparse24(x[:0].cuda(), scale[:0].cuda())[0].shape == (0, cols // 2)
    with pytest.raises(ValueError):
        ops.quantize_fp8_sparse24(x[:, :100].cuda(), scale.cuda())


@pytest.mark.parametrize("two_kernels", [False, True])
def test_c4b_bitmask_full(ops, orc, canary, two_kernels, request):
    """BASELINE config 4b at 4096 x 4096, Bernoulli(0.5) zero mask: the single-pass compress kernel (every block
    waits for the counts of the others) and the count + compaction pair."""
    from compressed_tensors_b200 import _lib as L

    L.lib().ctb_bitmask_force_two_kernels(L.i32(1 if two_kernels else 0))
    request.addfinalizer(lambda: L.lib().ctb_bitmask_force_two_kernels(L.i32(1)))
    g = torch.Generator().manual_seed(5)
    w = weights(4096, 4096, 5)
    w[torch.rand(4096, 4096, generator=g) < 0.5] = 0
    values, bitmask, row_offsets = orc.bitmask_compress(w)
    with canary():
        gv, gb, gr = ops.bitmask_compress(w.cuda())
        gd = ops.bitmask_decompress(gv, gb, w.shape)
    assert_bit_equal(gb.cpu(), bitmask, "bitmask")
    assert_bit_equal(gr.cpu(), row_offsets, "row offsets")
    assert_bit_equal(gv.cpu(), values, "values")
    assert_bit_equal(gd.cpu(), orc.bitmask_decompress(values, bitmask, w.shape), "decompressed")


def test_bitmask_large_and_repeated(ops, orc, request):
    """A tensor of many slabs (14336 x 4096: 3584 tiles, more than the grid holds at once) and twenty calls back to
    back on one workspace-sized scratch: the per-call ticket keeps stale counts of earlier calls from being taken."""
    from compressed_tensors_b200 import _lib as L

    L.lib().ctb_bitmask_force_two_kernels(L.i32(0))  # the single-pass kernel
    request.addfinalizer(lambda: L.lib().ctb_bitmask_force_two_kernels(L.i32(1)))
    g = torch.Generator().manual_seed(6)
    w = weights(14336, 4096, 6)
    w[torch.rand(14336, 4096, generator=g) < 0.7] = 0
    values, bitmask, row_offsets = orc.bitmask_compress(w)
    wd = w.cuda()
    for _ in range(3):
        gv, gb, gr = ops.bitmask_compress(wd)
        assert_bit_equal(gb.cpu(), bitmask, "bitmask")
        assert_bit_equal(gr.cpu(), row_offsets, "row offsets")
        assert_bit_equal(gv.cpu(), values, "values")
    small = [weights(64, 512, 100 + i) for i in range(20)]
    for i, t in enumerate(small):
        t[torch.rand(64, 512, generator=g) < 0.1 * (i % 10)] = 0
    outs = [ops._masked_compress(t.cuda(), None, sync=False) for t in small]
    torch.cuda.synchronize()
    for t, (v, b, r, n) in zip(small, outs):
        ev, eb, er = orc.bitmask_compress(t)
        assert int(n.item()) == ev.numel()
        assert_bit_equal(v[: ev.numel()].cpu(), ev, "values"), assert_bit_equal(b.cpu(), eb, "bitmask"), assert_bit_equal(r.cpu(), er, "row offsets")


def test_quantize_pack_batch_equals_oracle(ops, orc, canary):
    """The given-scale whole-shard entry point on a ragged table (tensors smaller than one unit, a partial last
    unit, a scale outside the reciprocal form's range): every tensor's words against the oracle."""
    shapes = [(8, 128), (4096, 4096), (1024, 4096), (33, 256), (4096, 14336)]
    ws = [weights(r, c, 60 + i) for i, (r, c) in enumerate(shapes)]
    want = []
    for i, w in enumerate(ws):
        mn, mx = orc.minmax(w, 1, 128)
        scale, zp = orc.calculate_qparams(mn, mx, qtype=orc.QINT, bits=4, symmetric=True)
        if i == 3:  # hand-made scales outside [2^-99, 2^99): the kernel's float routine takes these groups
            scale[5, 0], scale[7, 1] = 2.0 ** -110, 2.0 ** 100
        kw = dict(qtype=orc.QINT, bits=4, col_group=128, row_group=1, scale_row_stride=w.shape[1] // 128)
        want.append((scale, orc.pack_int32(orc.quantize(w, scale, zp, out_dtype=torch.int8, **kw), 4)))
    with canary():
        dw = [w.cuda() for w in ws]
        ds = [s.cuda() for s, _ in want]
        out = [torch.empty((w.shape[0], w.shape[1] // 8), dtype=torch.int32, device="cuda") for w in ws]
        ops.quantize_pack_int4_batch(ops.tensor_table(dw, out, ds, [tuple(w.shape) for w in ws]), torch.device("cuda", 0))
        torch.cuda.synchronize()
    for i, (o, (_, words)) in enumerate(zip(out, want)):
        assert_bit_equal(o.cpu(), words, f"tensor {i} {shapes[i]}")


def test_fp8_channel_batch_equals_oracle(ops, orc, canary):
    """The whole-shard FP8 entry points on a ragged table (a tensor smaller than one unit, a partial last unit, rows
    whose scale is outside the reciprocal form's range, NaN / Inf / signed zeros, zero points of zero and not):
    every tensor's codes and dequantized values against the oracle."""
    shapes = [(8, 128), (4096, 4096), (1024, 4096), (33, 264), (4096, 14336)]
    ws = [weights(r, c, 80 + i) for i, (r, c) in enumerate(shapes)]
    ws[3][0, :8] = torch.tensor([0.5, -0.5, float("inf"), -float("inf"), 0.0, -0.0, 1.0, -1.0]).to(torch.bfloat16)
    ws[3].view(torch.int16)[0, 8:12] = torch.tensor([0x7FC0, -64, 0x7F81, -1], dtype=torch.int16)
    ws[3][4] = -0.0
    scales, zps, want, deq = [], [], [], []
    for i, w in enumerate(ws):
        kw = dict(qtype=orc.QFLOAT, bits=8, col_group=w.shape[1], row_group=1, scale_row_stride=1)
        mn, mx = orc.minmax(torch.nan_to_num(w.float(), 0, 0, 0).to(torch.bfloat16), 1, w.shape[1])
        scale, zp = orc.calculate_qparams(mn, mx, qtype=orc.QFLOAT, bits=8, symmetric=True)
        if i == 3:
            scale[5, 0], scale[6, 0], scale[8, 0] = 2.0 ** -110, 2.0 ** 100, 2.0 ** -99
            zp = zp.to(torch.bfloat16)
            zp[9, 0], zp[10, 0] = 3.0, -1.5
        z = zp if i in (1, 3) else None  # a table may mix modules with and without a zero point
        q = orc.quantize(w, scale, z, out_dtype=torch.float8_e4m3fn, **kw)
        scales.append(scale)
        zps.append(None if z is None else z.to(torch.bfloat16))
        want.append(q)
        deq.append(orc.dequantize(q, scale, None, out_dtype=torch.bfloat16, **kw))
    dev = torch.device("cuda", 0)
    with canary():
        dw = [w.cuda() for w in ws]
        ds = [s.cuda().reshape(-1) for s in scales]
        dz = [None if z is None else z.cuda().reshape(-1) for z in zps]
        out = [torch.empty(w.shape, dtype=torch.float8_e4m3fn, device="cuda") for w in ws]
        back = [torch.empty(w.shape, dtype=torch.bfloat16, device="cuda") for w in ws]
        ops.quantize_fp8_channel_batch(ops.tensor_table(dw, out, ds, shapes), dz, dev)
        ops.dequantize_fp8_channel_batch(ops.tensor_table(out, back, ds, shapes), dev)
        torch.cuda.synchronize()
    for i in range(len(ws)):
        assert_bit_equal(out[i].cpu(), want[i], f"codes of tensor {i} {shapes[i]}")
        got, ref = back[i].cpu(), deq[i]
        nan = got.float().isnan() & ref.float().isnan()  # a NaN code decodes to a NaN; its payload is the platform's
        assert_bit_equal(torch.where(nan, torch.zeros_like(got), got), torch.where(nan, torch.zeros_like(ref), ref),
                         f"dequantized tensor {i} {shapes[i]}")


def test_nvfp4_batch_equals_oracle(ops, orc, canary):
    """The whole-shard NVFP4 entry points on a ragged table (a tensor smaller than one unit, partial last units, a
    different global scale per tensor so that the decompress kernel's scale table is rebuilt, zero points present and
    absent, signed zeros and values beyond the grid): codes and dequantized values against the oracle."""
    shapes = [(8, 128), (4096, 4096), (1024, 4096), (33, 272), (14336, 4096)]
    ws = [weights(r, c, 90 + i, std=0.02 * (1 + i)) for i, (r, c) in enumerate(shapes)]
    ws[3][0, :8] = torch.tensor([0.5, -0.5, 3.0, -3.0, 0.0, -0.0, 1.0, -1.0]).to(torch.bfloat16)
    ws[3][4] = -0.0
    scales, gss, zps, want, deq = [], [], [], [], []
    for i, w in enumerate(ws):
        kw = dict(qtype=orc.QFLOAT, bits=4, col_group=16, row_group=1, scale_row_stride=w.shape[1] // 16)
        tmn, tmx = orc.minmax(w, w.shape[0], w.shape[1])
        gs = orc.generate_gparam(tmn, tmx)
        mn, mx = orc.minmax(w, 1, 16)
        scale, zp = orc.calculate_qparams(mn, mx, qtype=orc.QFLOAT, bits=4, symmetric=True, global_scale=gs)
        z = zp if i in (1, 3) else None
        if i == 3:  # a zero point other than zero and infinite inputs take the kernel's general routine
            z = z.clone()
            z[9, 0], z[10, 3] = 1.0, -0.5
            w[11, 5], w[11, 40] = float("inf"), -float("inf")
        packed = orc.pack_fp4(orc.quantize(w, scale, z, out_dtype=torch.bfloat16, global_scale=gs, **kw))
        scales.append(scale)
        gss.append(gs)
        zps.append(z)
        want.append(packed)
        deq.append(orc.dequantize(orc.unpack_fp4(packed, *w.shape), scale, None, out_dtype=torch.bfloat16, global_scale=gs, **kw))
    dev = torch.device("cuda", 0)
    with canary():
        dw = [w.cuda() for w in ws]
        ds = [s.cuda() for s in scales]
        dg = [g.cuda().reshape(1) for g in gss]
        dz = [None if z is None else z.cuda() for z in zps]
        out = [torch.empty((r, c // 2), dtype=torch.uint8, device="cuda") for r, c in shapes]
        back = [torch.empty((r, c), dtype=torch.bfloat16, device="cuda") for r, c in shapes]
        ops.quantize_fp4_g16_batch(ops.tensor_table(dw, out, ds, shapes), dg, dz, dev)
        ops.dequantize_fp4_g16_batch(ops.tensor_table(out, back, ds, shapes), dg, dev)
        torch.cuda.synchronize()
    for i in range(len(ws)):
        assert_bit_equal(out[i].cpu(), want[i], f"packed codes of tensor {i} {shapes[i]}")
        assert_bit_equal(back[i].cpu(), deq[i], f"dequantized tensor {i} {shapes[i]}")
