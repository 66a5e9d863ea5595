"""CUDA kernels (through the C ABI) against the reference's own outputs stored in tests/golden/."""
import pytest
import torch

from tests.helpers import assert_bit_equal, assert_value_equal

pytestmark = pytest.mark.gpu

INT_CASES = [
    "w4_sym_g128_bf16", "w4_asym_g128_bf16", "w4_sym_g32_bf16", "w8_sym_g128_bf16",
    "w8_sym_channel_bf16", "w8_asym_channel_bf16", "w4_sym_tensor_bf16", "w4_sym_g128_fp32",
    "w4_asym_g64_fp16", "w4_sym_channel_fp32",
]


@pytest.fixture(scope="module")
def ops():
    from compressed_tensors_b200 import ops as o
    return o


def dev(t):
    return t.cuda()


def layout(x, scale, group):
    cols = x.shape[-1]
    if scale.numel() == 1:
        return cols, 0
    g = group if group else cols
    return g, cols // g


@pytest.mark.parametrize("name", INT_CASES)
def test_int_quant(golden, ops, name):
    d = golden("int_quant")[name]
    x, scale, zp = dev(d["x"]), dev(d["scale"]), dev(d["zp"])
    bits, sym, group = int(d["bits"]), bool(d["sym"]), int(d["group"])
    cg, srs = layout(x, scale, group)
    kw = dict(qtype=ops.QINT, bits=bits, col_group=cg, row_group=1, scale_row_stride=srs)

    mn, mx = ops.minmax(x, x.shape[0] if scale.numel() == 1 else 1, cg)
    assert_value_equal(mn.reshape(d["min"].shape).cpu(), d["min"], "min")
    assert_value_equal(mx.reshape(d["max"].shape).cpu(), d["max"], "max")
    s, z = ops.calculate_qparams(dev(d["min"]), dev(d["max"]), qtype=ops.QINT, bits=bits, symmetric=sym)
    assert_bit_equal(s.reshape(scale.shape).cpu(), d["scale"], "scale")
    assert_bit_equal(z.reshape(zp.shape).cpu(), d["zp"], "zero point")

    q8 = ops.quantize(x, scale, zp, out_dtype=torch.int8, **kw)
    assert_bit_equal(q8.cpu(), d["q_int8"], "int8 codes")
    assert_bit_equal(ops.quantize(x, scale, zp, out_dtype=d["q_float"].dtype, **kw).cpu(), d["q_float"], "float codes")
    packed = ops.quantize(x, scale, zp, codec="pack32", **kw)
    assert_bit_equal(packed.cpu(), d["packed"], "fused quantize+pack words")
    assert_bit_equal(ops.pack_int32(q8, bits).cpu(), d["packed"], "pack_to_int32")
    assert_bit_equal(ops.unpack_int32(packed, bits, x.shape).cpu(), d["unpacked"], "unpack_from_int32")
    assert_bit_equal(ops.dequantize(q8, scale, zp, out_dtype=d["dequant"].dtype, **kw).cpu(), d["dequant"], "dequant")
    fused = ops.dequantize(packed, scale, zp, out_dtype=d["dequant"].dtype, codec="pack32", cols=x.shape[1], **kw)
    assert_bit_equal(fused.cpu(), d["dequant"], "fused unpack+dequant")
    assert_bit_equal(ops.fake_quantize(x, scale, zp, out_dtype=d["fake"].dtype, **kw).cpu(), d["fake"], "fake quant")
    if "c_weight_zero_point" in d:
        pz = ops.pack_int32(zp, bits, packed_dim=0).contiguous()
        assert_bit_equal(pz.cpu(), d["c_weight_zero_point"], "packed zero point")
        back = ops.unpack_int32(pz, bits, zp.shape, packed_dim=0)
        assert_bit_equal(back.contiguous().cpu(), d["zp"], "unpacked zero point")
    if sym and scale.numel() > 1 and cg <= 256 and cg % 8 == 0 and x.dtype == torch.bfloat16:
        w, sc = ops.absmax_quantize(x, qtype=ops.QINT, bits=bits, col_group=cg, codec="pack32")
        assert_bit_equal(sc.cpu().reshape(d["scale"].shape), d["scale"], "fused calibrate: scale")
        assert_bit_equal(w.cpu(), d["packed"], "fused calibrate: words")


def test_int_actorder(golden, ops):
    d = golden("int_quant")["w4_sym_g64_actorder"]
    x, scale, zp, g_idx = dev(d["x"]), dev(d["scale"]), dev(d["zp"]), dev(d["g_idx"])
    kw = dict(qtype=ops.QINT, bits=4, col_group=64, row_group=1, scale_row_stride=scale.shape[1], g_idx=g_idx)
    q8 = ops.quantize(x, scale, zp, out_dtype=torch.int8, **kw)
    assert_bit_equal(q8.cpu(), d["q_int8"], "codes")
    assert_bit_equal(ops.dequantize(q8, scale, zp, out_dtype=torch.bfloat16, **kw).cpu(), d["dequant"], "dequant")
    assert_bit_equal(ops.fake_quantize(x, scale, zp, out_dtype=torch.bfloat16, **kw).cpu(), d["fake"], "fake")


def test_pack_known_words(golden, ops):
    g = golden("int_quant")
    for k in ("pack_known_4_8", "pack_known_8_4", "pack_known_4_3", "pack_known_2_20"):
        d = g[k]
        bits = int(d["bits"])
        assert_bit_equal(ops.pack_int32(dev(d["value"]), bits).cpu(), d["packed"], k)
        assert_bit_equal(ops.unpack_int32(dev(d["packed"]), bits, d["value"].shape).cpu(), d["value"], k)
    d = g["pack_dim0"]
    got = ops.pack_int32(dev(d["value"]), 4, packed_dim=0)
    assert_bit_equal(got.contiguous().cpu(), d["packed"], "packed_dim=0")
    assert_bit_equal(ops.unpack_int32(got, 4, d["value"].shape, packed_dim=0).contiguous().cpu(), d["unpacked"], "unpack dim 0")


@pytest.mark.parametrize("name", ["channel_bf16", "channel_bf16_f32scale", "channel_fp16", "channel_fp32",
                                  "tensor_bf16", "token_bf16", "block_bf16"])
def test_fp8(golden, ops, name):
    d = golden("fp8_quant")[name]
    x, scale, zp = dev(d["x"]), dev(d["scale"]), dev(d["zp"])
    cols = x.shape[-1]
    if name == "block_bf16":
        kw = dict(col_group=64, row_group=16, scale_row_stride=scale.shape[1])
    elif scale.numel() == 1:
        kw = dict(col_group=cols, row_group=1, scale_row_stride=0)
    else:
        kw = dict(col_group=cols, row_group=1, scale_row_stride=1)
    kw.update(qtype=ops.QFLOAT, bits=8)
    q = ops.quantize(x, scale, zp, out_dtype=torch.float8_e4m3fn, **kw)
    assert_bit_equal(q.cpu(), d["q"], "e4m3 codes")
    if "q_float" in d:
        assert_bit_equal(ops.quantize(x, scale, zp, out_dtype=d["q_float"].dtype, **kw).cpu(), d["q_float"], "float codes")
    assert_bit_equal(ops.dequantize(q, scale, zp, out_dtype=d["dequant"].dtype, **kw).cpu(), d["dequant"], "dequant")
    assert_bit_equal(ops.fake_quantize(x, scale, zp, out_dtype=d["fake"].dtype, **kw).cpu(), d["fake"], "fake")
    rg = 16 if name == "block_bf16" else (x.numel() // cols if scale.numel() == 1 else 1)
    src = x.to(scale.dtype) if scale.dtype != x.dtype else x
    mn, mx = ops.minmax(src, rg, kw["col_group"])
    s, z = ops.calculate_qparams(mn, mx, qtype=ops.QFLOAT, bits=8, symmetric=True)
    assert_bit_equal(s.reshape(scale.shape).cpu(), d["scale"], "scale")
    assert_bit_equal(z.reshape(zp.shape).cpu(), d["zp"], "zp")
    if name in ("channel_bf16", "token_bf16"):
        qq, sc = ops.absmax_quantize(x, qtype=ops.QFLOAT, bits=8, col_group=cols, codec="dtype", out_dtype=torch.float8_e4m3fn)
        assert_bit_equal(sc.reshape(scale.shape).cpu(), d["scale"], "fused calibrate: scale")
        assert_bit_equal(qq.cpu(), d["q"], "fused calibrate: codes")


def test_e4m3_rounding_probe(golden, ops):
    d = golden("fp8_quant")["e4m3_probe"]
    x = dev(d["x"])
    q = ops.quantize(x, dev(d["scale"]), None, out_dtype=torch.float8_e4m3fn, qtype=ops.QFLOAT, bits=8,
                     col_group=x.shape[1], row_group=1, scale_row_stride=0)
    assert_bit_equal(q.cpu(), d["q"])


@pytest.mark.parametrize("name", ["a", "b"])
def test_nvfp4(golden, ops, name):
    d = golden("nvfp4")[name]
    x, scale, gs = dev(d["x"]), dev(d["scale"]), dev(d["global_scale"])
    rows, cols = x.shape
    mn, mx = ops.minmax(x, rows, cols)
    assert_value_equal(mn.reshape(1).cpu(), d["min"]), assert_value_equal(mx.reshape(1).cpu(), d["max"])
    assert_bit_equal(ops.generate_gparam(mn, mx).cpu(), d["global_scale"], "global scale")
    gmn, gmx = ops.minmax(x, 1, 16)
    s, z = ops.calculate_qparams(gmn, gmx, qtype=ops.QFLOAT, bits=4, symmetric=True, global_scale=gs)
    assert_bit_equal(s.cpu(), d["scale"], "local scales")
    assert_bit_equal(z.cpu(), d["zp"], "zp")
    kw = dict(qtype=ops.QFLOAT, bits=4, col_group=16, row_group=1, scale_row_stride=cols // 16, global_scale=gs)
    q = ops.quantize(x, scale, None, out_dtype=torch.bfloat16, **kw)
    assert_bit_equal(q.cpu(), d["q"], "e2m1 values (incl. sign of zero)")
    assert_bit_equal(ops.pack_fp4(q).cpu(), d["packed"], "pack_fp4_to_uint8")
    packed = ops.quantize(x, scale, None, codec="fp4x2", **kw)
    assert_bit_equal(packed.cpu(), d["packed"], "fused quantize+pack bytes")
    un = ops.unpack_fp4(packed, rows, cols)
    assert_bit_equal(un.cpu(), d["unpacked"], "unpack_fp4_from_uint8")
    assert_bit_equal(ops.dequantize(un, scale, None, out_dtype=torch.bfloat16, **kw).cpu(), d["dequant"], "dequant")
    assert_bit_equal(ops.dequantize(packed, scale, None, out_dtype=torch.bfloat16, codec="fp4x2", **kw).cpu(), d["dequant"], "fused unpack+dequant")
    assert_bit_equal(ops.fake_quantize(x, scale, None, out_dtype=torch.bfloat16, **kw).cpu(), d["fake"], "fake")
    pk, sc = ops.absmax_quantize(x, qtype=ops.QFLOAT, bits=4, col_group=16, codec="fp4x2", global_scale=gs)
    assert_bit_equal(sc.cpu(), d["scale"], "fused calibrate: scales")
    assert_bit_equal(pk.cpu(), d["packed"], "fused calibrate: bytes")


def test_e2m1_threshold_probe(golden, ops):
    d = golden("nvfp4")["e2m1_probe"]
    x = dev(d["x"])
    kw = dict(qtype=ops.QFLOAT, bits=4, col_group=16, row_group=1, scale_row_stride=x.shape[1] // 16,
              global_scale=dev(d["global_scale"]))
    q = ops.quantize(x, dev(d["scale"]), None, out_dtype=torch.float32, **kw)
    assert_bit_equal(q.cpu(), d["q"])
    assert_bit_equal(ops.pack_fp4(q).cpu(), d["packed"])
    # the hardware e2m1 convert (vec8 tier) on the same sweep, from bf16-representable inputs
    xb = x.to(torch.bfloat16)
    ref = ops.pack_fp4(ops.quantize(xb.float(), dev(d["scale"]), None, out_dtype=torch.float32, **kw))
    assert_bit_equal(ops.quantize(xb, dev(d["scale"]), None, codec="fp4x2", **kw).cpu(), ref.cpu(), "cvt.e2m1x2 vs thresholds")


@pytest.mark.parametrize("tag", ["bf16", "fp16", "fp32", "e4m3"])
@pytest.mark.parametrize("cols", [64, 13])
def test_bitmask(golden, ops, tag, cols):
    d = golden("sparse")[f"bitmask_{tag}_{cols}"]
    x = dev(d["x"])
    values, bitmask, row_offsets = ops.bitmask_compress(x)
    assert_bit_equal(values.cpu(), d["values"], "values")
    assert_bit_equal(bitmask.cpu(), d["bitmask"], "bitmask")
    assert_bit_equal(row_offsets.cpu(), d["row_offsets"], "row offsets")
    assert_bit_equal(ops.bitmask_decompress(values, bitmask, x.shape).cpu(), d["dense"], "dense")
    mask = ops.unpack_bitmasks(bitmask, x.shape)
    assert_bit_equal(ops.pack_bitmasks(mask).cpu(), d["bitmask"])


@pytest.mark.parametrize("tag", ["bf16", "fp32", "int8", "e4m3"])
def test_sparse24(golden, ops, tag):
    d = golden("sparse")[f"s24_{tag}"]
    x = dev(d["x"])
    assert_bit_equal(ops.sparse24_mask(x).cpu(), d["mask"], "2:4 keep mask")
    values, bitmask = ops.sparse24_compress(x)
    assert_bit_equal(values.cpu(), d["values"], "values")
    assert_bit_equal(bitmask.cpu(), d["bitmask"], "bitmask")
    assert_bit_equal(ops.bitmask_decompress(values, bitmask, x.shape).cpu(), d["dense"], "dense")


def test_sparse24_all_weak_orderings(golden, ops):
    d = golden("sparse")["s24_rank_patterns"]
    assert_bit_equal(ops.sparse24_mask(dev(d["ranks"].float())).cpu(), d["mask"])
    assert_bit_equal(ops.sparse24_mask(dev(d["ranks"])).cpu(), d["mask_int8"])
    assert_bit_equal(ops.sparse24_mask(dev(d["ranks"].to(torch.bfloat16))).cpu(), d["mask_bf16"])


def test_hadamard(golden, ops):
    g = golden("hadamard")
    for name, d in g.items():
        if not (name.startswith("hadamard_") or name.startswith("random_")):
            continue
        m = d["matrix"]
        n = m.shape[0]
        signs = dev(m[:, 0].clone())
        side = 0 if "weight_input" in name else 1
        out = ops.hadamard(dev(d["w"]), n, signs=signs, inverse="_inv_" in name, side=side, precision=torch.float64)
        if d["w"].dtype == torch.bfloat16:
            assert_bit_equal(out.cpu(), d["out"], name)
        else:
            torch.testing.assert_close(out.cpu(), d["out"], rtol=1e-6, atol=1e-7, msg=name)
        fast = ops.hadamard(dev(d["w"]), n, signs=signs, inverse="_inv_" in name, side=side, precision=torch.float32)
        # fp32 accumulation: rel-err <= 1e-3 against the float64 result (norm-wise)
        err = (fast.double().cpu() - d["out"].double()).norm() / d["out"].double().norm()
        assert err <= 1e-3, (name, float(err))


def test_mxfp4_scale_helpers_every_input(golden, ops):
    """mxfp4_utils.py on all 65536 bf16 bit patterns and all 256 exponent bytes, through the host mirror"""
    from compressed_tensors_b200.quantization.utils import convert_mxfp4_exp_scale, generate_mxfp4_scales, round_to_power_2

    d = golden("mxfp4")
    x = torch.arange(65536, dtype=torch.int32).to(torch.uint16).view(torch.bfloat16).cuda()
    assert torch.equal(round_to_power_2(x).view(torch.uint16).cpu(), d["all_bf16"]["round_pow2_bits"])
    assert torch.equal(generate_mxfp4_scales(x).cpu(), d["all_bf16"]["scales"])
    e = torch.arange(256, dtype=torch.int32).to(torch.uint8).cuda()
    for key, dt in (("bf16", torch.bfloat16), ("f16", torch.float16), ("f32", torch.float32)):
        assert_bit_equal(convert_mxfp4_exp_scale(e, dt).cpu(), d["all_exponents"][key], key)


def test_fp4_pack_every_16bit_input(golden, ops):
    """pack_fp4_to_uint8 on all 65536 bf16 and f16 bit patterns and a float32 sweep; unpack on every byte; both the
    8-values-per-thread kernels and (odd element counts, unaligned views) the scalar ones"""
    d = golden("fp4_pack_all")
    bits = torch.arange(65536, dtype=torch.int32).to(torch.uint16).reshape(256, 256)
    for key, dt in (("bf16", torch.bfloat16), ("f16", torch.float16)):
        x = bits.view(dt).cuda()
        assert torch.equal(ops.pack_fp4(x).cpu(), d[key + "_packed"]), key
        assert torch.equal(ops.pack_fp4(x[:, :254].contiguous()).cpu(), d[key + "_packed"][:, :127]), key + " scalar kernel"
    assert torch.equal(ops.pack_fp4(d["f32"].cuda()).cpu(), d["f32_packed"])
    assert torch.equal(ops.pack_fp4(d["f32"][:, :126].contiguous().cuda()).cpu(), d["f32_packed"][:, :63])
    every_byte = torch.arange(256, dtype=torch.int32).to(torch.uint8).reshape(16, 16).cuda()
    for key, dt in (("bf16", torch.bfloat16), ("f16", torch.float16), ("f32", torch.float32)):
        assert_bit_equal(ops.unpack_fp4(every_byte, 16, 32, dtype=dt).cpu(), d["unpacked_" + key], key)
        assert_bit_equal(ops.unpack_fp4(every_byte[:1, :3].contiguous(), 1, 6, dtype=dt).cpu(), d["unpacked_" + key].reshape(-1)[:6].reshape(1, 6), key)


def test_minmax_tiles_match_oracle(ops):
    """BLOCK-strategy min / max: tiles whose rows are whole 16-byte chunks (vector kernel) and tiles that are not"""
    from oracle import ref as orc

    g = torch.Generator().manual_seed(21)
    for dt in (torch.bfloat16, torch.float16, torch.float32):
        x = torch.randn(256, 384, generator=g).to(dt)
        for rg, cg in ((128, 128), (64, 32), (16, 8), (256, 96), (2, 384), (32, 4), (8, 12)):
            mn, mx = ops.minmax(x.cuda(), rg, cg)
            wmn, wmx = orc.minmax(x, rg, cg)
            assert_bit_equal(mn.cpu(), wmn, f"min {dt} {rg}x{cg}")
            assert_bit_equal(mx.cpu(), wmx, f"max {dt} {rg}x{cg}")


def test_empty_and_degenerate_tensors(ops):
    """a tensor with no elements has no storage (null pointer): every codec returns an empty result of the right
    shape instead of raising, as the reference's tensor expressions do; all-zero and all-dense tensors round-trip"""
    dev = "cuda"
    e16 = torch.empty((0, 16), dtype=torch.bfloat16, device=dev)
    v, b, r = ops.bitmask_compress(e16)
    assert (tuple(v.shape), tuple(b.shape), tuple(r.shape)) == ((0,), (0, 2), (0,))
    assert tuple(ops.bitmask_decompress(v, b, (0, 16)).shape) == (0, 16)
    assert tuple(ops.sparse24_mask(e16).shape) == (0, 16)
    v, b = ops.sparse24_compress(e16)
    assert (tuple(v.shape), tuple(b.shape)) == ((0, 8), (0, 2))
    assert tuple(ops.sparse24_decompress(v, b, (0, 16)).shape) == (0, 16)
    sp, meta = ops.cutlass24_compress(torch.empty((0, 64), dtype=torch.int8, device=dev))
    assert (tuple(sp.shape), tuple(meta.shape)) == ((0, 32), (0, 4))
    assert ops.mxfp4_generate_scales(torch.empty((0,), dtype=torch.bfloat16, device=dev)).numel() == 0
    q, s = ops.absmax_quantize(torch.empty((0, 128), dtype=torch.bfloat16, device=dev), qtype=ops.QINT, bits=4, col_group=128, codec="pack32")
    assert (tuple(q.shape), tuple(s.shape)) == ((0, 16), (0, 1))
    kw = dict(qtype=ops.QINT, bits=4, col_group=128, scale_row_stride=1)
    assert tuple(ops.quantize(torch.empty((0, 128), dtype=torch.bfloat16, device=dev), s, None, codec="pack32", **kw).shape) == (0, 16)
    assert tuple(ops.dequantize(q, s, None, out_dtype=torch.bfloat16, codec="pack32", cols=128, **kw).shape) == (0, 128)
    assert tuple(ops.hadamard(torch.empty((0, 128), dtype=torch.bfloat16, device=dev), 128).shape) == (0, 128)
    z = torch.zeros((512, 4096), dtype=torch.bfloat16, device=dev)
    v, b, r = ops.bitmask_compress(z)
    assert v.numel() == 0 and int(b.sum()) == 0 and int(r.sum()) == 0
    assert torch.equal(ops.bitmask_decompress(v, b, (512, 4096)), z)
    o = torch.ones((512, 4096), dtype=torch.bfloat16, device=dev)
    v, b, r = ops.bitmask_compress(o)
    assert v.numel() == o.numel() and bool((b == 255).all()) and int(r[-1]) == 511 * 4096
    assert torch.equal(ops.bitmask_decompress(v, b, (512, 4096)), o)



def test_generate_gparam_sweep(golden):
    """The device kernel against the reference on every 5th positive bf16 / fp16 maximum, the float32 sample and
    minima that dominate (the scalar-on-the-left division of the reference rounds twice)."""
    from compressed_tensors_b200 import ops

    g = golden("gparam_all")
    for tag in ("bf16", "f16", "f32"):
        mx, want = g[tag]["max"][::5].cuda(), g[tag]["global_scale"][::5]
        zero = torch.zeros((), dtype=mx.dtype, device="cuda")
        got = torch.cat([ops.generate_gparam(zero, m) for m in mx])
        assert_bit_equal(got.cpu(), want, f"global scale, {tag} maxima")
    mn, want = g["neg"]["min"].cuda(), g["neg"]["global_scale"]
    got = torch.cat([ops.generate_gparam(m, -m / 2) for m in mn])
    assert_bit_equal(got.cpu(), want, "global scale, dominated by the minimum")
