"""Pins the CPU oracle against fixtures produced by the reference implementation
(tests/golden/make_golden.py).  Runs without a GPU."""
import pytest
import torch

from oracle import ref as orc
from tests.helpers import assert_bit_equal

INT_CASES = [
    "w4_sym_g128_bf16", "w4_asym_g128_bf16", "w4_sym_g32_bf16", "w8_sym_g128_bf16",
    "w8_sym_channel_bf16", "w8_asym_channel_bf16", "w4_sym_tensor_bf16", "w4_sym_g128_fp32",
    "w4_asym_g64_fp16", "w4_sym_channel_fp32",
]


def layout(x, scale, group):
    """(col_group, scale_row_stride) of a scale tensor against x viewed as [rows, cols]."""
    cols = x.shape[-1]
    if scale.numel() == 1:
        return cols, 0
    g = group if group else cols
    return g, cols // g


@pytest.mark.parametrize("name", INT_CASES)
def test_int_quant(golden, name):
    d = golden("int_quant")[name]
    x, scale, zp = d["x"], d["scale"], d["zp"]
    bits, sym, group = int(d["bits"]), bool(d["sym"]), int(d["group"])
    cg, srs = layout(x, scale, group)
    kw = dict(qtype=orc.QINT, bits=bits, col_group=cg, row_group=1, scale_row_stride=srs)

    mn, mx = orc.minmax(x, x.shape[0] if scale.numel() == 1 else 1, cg)
    assert_bit_equal(mn.reshape(d["min"].shape), d["min"], "min")
    assert_bit_equal(mx.reshape(d["max"].shape), d["max"], "max")
    s, z = orc.calculate_qparams(d["min"], d["max"], qtype=orc.QINT, bits=bits, symmetric=sym)
    assert_bit_equal(s.reshape(scale.shape), scale, "scale")
    assert_bit_equal(z.reshape(zp.shape), zp, "zero point")

    q8 = orc.quantize(x, scale, zp, out_dtype=torch.int8, **kw)
    assert_bit_equal(q8, d["q_int8"], "int8 codes")
    assert_bit_equal(orc.quantize(x, scale, zp, out_dtype=d["q_float"].dtype, **kw), d["q_float"], "float codes")
    packed = orc.pack_int32(q8, bits)
    assert_bit_equal(packed, d["packed"], "packed words")
    assert_bit_equal(packed, d["c_weight_packed"], "compressor words")
    assert_bit_equal(orc.unpack_int32(packed, bits, x.shape), d["unpacked"], "unpacked")
    assert_bit_equal(orc.dequantize(q8, scale, zp, out_dtype=d["dequant"].dtype, **kw), d["dequant"], "dequant")
    assert_bit_equal(d["dequant_noargs"], d["dequant"], "strategy inference")
    assert_bit_equal(orc.fake_quantize(x, scale, zp, out_dtype=d["fake"].dtype, **kw), d["fake"], "fake quant")
    assert_bit_equal(d["decompressed"], d["dequant"], "decompress_weight == dequantize(unpack)")
    assert d["c_weight_shape"].dtype == torch.int64 and d["c_weight_shape"].tolist() == list(x.shape)
    if "c_weight_zero_point" in d:
        got = orc.pack_int32(zp.t().contiguous(), bits).t().contiguous()
        assert_bit_equal(got, d["c_weight_zero_point"], "packed zero point")


def test_int_actorder(golden):
    d = golden("int_quant")["w4_sym_g64_actorder"]
    x, scale, zp, g_idx = d["x"], d["scale"], d["zp"], d["g_idx"]
    kw = dict(qtype=orc.QINT, bits=4, col_group=64, row_group=1, scale_row_stride=scale.shape[1], g_idx=g_idx)
    q8 = orc.quantize(x, scale, zp, out_dtype=torch.int8, **kw)
    assert_bit_equal(q8, d["q_int8"], "codes")
    assert_bit_equal(orc.dequantize(q8, scale, zp, out_dtype=torch.bfloat16, **kw), d["dequant"], "dequant")
    assert_bit_equal(orc.fake_quantize(x, scale, zp, out_dtype=torch.bfloat16, **kw), d["fake"], "fake")


def test_pack_known_words(golden):
    g = golden("int_quant")
    # the literal words asserted by the reference's own test-suite
    assert g["pack_known_4_8"]["packed"].tolist() == [[1985229328]]
    assert g["pack_known_8_4"]["packed"].tolist() == [[-2071756159]]
    for k in ("pack_known_4_8", "pack_known_8_4", "pack_known_4_3", "pack_known_2_20"):
        d = g[k]
        bits = int(d["bits"])
        assert_bit_equal(orc.pack_int32(d["value"], bits), d["packed"], k)
        assert_bit_equal(orc.unpack_int32(d["packed"], bits, d["value"].shape), d["value"], k)
    d = g["pack_dim0"]
    got = orc.pack_int32(d["value"].t().contiguous(), 4).t().contiguous()
    assert_bit_equal(got, d["packed"], "packed_dim=0")
    back = orc.unpack_int32(got.t().contiguous(), 4, (d["value"].shape[1], d["value"].shape[0])).t()
    assert_bit_equal(back.contiguous(), d["unpacked"], "unpack packed_dim=0")


@pytest.mark.parametrize("name", ["channel_bf16", "channel_bf16_f32scale", "channel_fp16", "channel_fp32",
                                  "tensor_bf16", "token_bf16", "block_bf16"])
def test_fp8(golden, name):
    d = golden("fp8_quant")[name]
    x, scale, zp = d["x"], d["scale"], d["zp"]
    cols = x.shape[-1]
    if name == "block_bf16":
        kw = dict(col_group=64, row_group=16, scale_row_stride=scale.shape[1])
    elif scale.numel() == 1:
        kw = dict(col_group=cols, row_group=1, scale_row_stride=0)
    else:
        kw = dict(col_group=cols, row_group=1, scale_row_stride=1)
    kw.update(qtype=orc.QFLOAT, bits=8)
    # the reference adds the (all-zero) zero point, which turns a -0.0 quotient into +0.0
    q = orc.quantize(x, scale, zp, out_dtype=torch.float8_e4m3fn, **kw)
    assert_bit_equal(q, d["q"], "e4m3 codes")
    if "q_float" in d:
        assert_bit_equal(orc.quantize(x, scale, zp, out_dtype=d["q_float"].dtype, **kw), d["q_float"], "float codes")
    assert_bit_equal(orc.dequantize(q, scale, zp, out_dtype=d["dequant"].dtype, **kw), d["dequant"], "dequant")
    assert_bit_equal(orc.fake_quantize(x, scale, zp, out_dtype=d["fake"].dtype, **kw), d["fake"], "fake")
    # qparams
    rg = 16 if name == "block_bf16" else (x.numel() // cols if scale.numel() == 1 else 1)
    src = x.to(scale.dtype) if scale.dtype != x.dtype else x
    mn, mx = orc.minmax(src, rg, kw["col_group"])
    s, z = orc.calculate_qparams(mn, mx, qtype=orc.QFLOAT, bits=8, symmetric=True)
    assert_bit_equal(s.reshape(scale.shape), scale, "scale")
    assert_bit_equal(z.reshape(zp.shape), zp, "zp")
    if "decompressed" in d:
        assert_bit_equal(d["c_weight"], d["q"], "naive compressor")
        assert_bit_equal(d["decompressed"], d["dequant"], "naive decompress")


def test_fp8_token_2d_collapses_to_one_scale(golden):
    d = golden("fp8_quant")["token_2d"]
    assert d["scale"].numel() == 1
    mn, mx = orc.minmax(d["x"], d["x"].shape[0], d["x"].shape[1])
    s, _ = orc.calculate_qparams(mn, mx, qtype=orc.QFLOAT, bits=8, symmetric=True)
    assert_bit_equal(s.reshape(d["scale"].shape), d["scale"])


def test_e4m3_rounding_probe(golden):
    d = golden("fp8_quant")["e4m3_probe"]
    x = d["x"]
    q = orc.quantize(x, d["scale"], None, out_dtype=torch.float8_e4m3fn, qtype=orc.QFLOAT, bits=8,
                     col_group=x.shape[1], row_group=1, scale_row_stride=0)
    assert_bit_equal(q, d["q"])


@pytest.mark.parametrize("name", ["a", "b"])
def test_nvfp4(golden, name):
    d = golden("nvfp4")[name]
    x, scale, gs = d["x"], d["scale"], d["global_scale"]
    rows, cols = x.shape
    mn, mx = orc.minmax(x, rows, cols)
    assert_bit_equal(mn.reshape(1), d["min"]), assert_bit_equal(mx.reshape(1), d["max"])
    assert_bit_equal(orc.generate_gparam(mn, mx), gs, "global scale")
    gmn, gmx = orc.minmax(x, 1, 16)
    assert_bit_equal(gmn, d["gmin"]), assert_bit_equal(gmx, d["gmax"])
    s, z = orc.calculate_qparams(gmn, gmx, qtype=orc.QFLOAT, bits=4, symmetric=True, global_scale=gs)
    assert_bit_equal(s, scale, "local scales")
    assert_bit_equal(z, d["zp"], "zp")
    kw = dict(qtype=orc.QFLOAT, bits=4, col_group=16, row_group=1, scale_row_stride=cols // 16, global_scale=gs)
    q = orc.quantize(x, scale, None, out_dtype=torch.bfloat16, **kw)
    assert_bit_equal(q, d["q"], "e2m1 values (incl. sign of zero)")
    packed = orc.pack_fp4(q)
    assert_bit_equal(packed, d["packed"], "packed bytes")
    assert_bit_equal(packed, d["c_weight_packed"], "compressor bytes")
    un = orc.unpack_fp4(packed, rows, cols)
    assert_bit_equal(un, d["unpacked"], "unpacked")
    deq = orc.dequantize(un, scale, None, out_dtype=torch.bfloat16, **kw)
    assert_bit_equal(deq, d["dequant"], "dequant")
    assert_bit_equal(d["decompressed"], d["dequant"])
    assert_bit_equal(orc.fake_quantize(x, scale, None, out_dtype=torch.bfloat16, **kw), d["fake"], "fake")


def test_e2m1_threshold_probe(golden):
    d = golden("nvfp4")["e2m1_probe"]
    x = d["x"]
    q = orc.quantize(x, d["scale"], None, out_dtype=torch.float32, qtype=orc.QFLOAT, bits=4, col_group=16,
                     row_group=1, scale_row_stride=x.shape[1] // 16, global_scale=d["global_scale"])
    assert_bit_equal(q, d["q"])
    assert_bit_equal(orc.pack_fp4(q), d["packed"])
    # the sign nibble cases called out by the reference's fp4 test
    one = torch.tensor([[-0.1, -0.0]], dtype=torch.float32)
    s = torch.ones(1, 1, dtype=torch.float8_e4m3fn)
    qq = orc.quantize(torch.nn.functional.pad(one, (0, 14)), s, None, out_dtype=torch.float32, qtype=orc.QFLOAT,
                      bits=4, col_group=16, row_group=1, scale_row_stride=1, global_scale=torch.ones(1))
    assert orc.pack_fp4(qq)[0, 0].item() == 0x08


@pytest.mark.parametrize("tag", ["bf16", "fp16", "fp32", "e4m3"])
@pytest.mark.parametrize("cols", [64, 13])
def test_bitmask(golden, tag, cols):
    d = golden("sparse")[f"bitmask_{tag}_{cols}"]
    values, bitmask, row_offsets = orc.bitmask_compress(d["x"])
    assert_bit_equal(values, d["values"], "values")
    assert_bit_equal(bitmask, d["bitmask"], "bitmask")
    assert_bit_equal(row_offsets, d["row_offsets"], "row offsets")
    assert_bit_equal(orc.bitmask_decompress(values, bitmask, d["x"].shape), d["dense"], "dense")
    mask = orc.unpack_bitmasks(bitmask, d["x"].shape)
    assert_bit_equal(orc.pack_bitmasks(mask), bitmask)


@pytest.mark.parametrize("tag", ["bf16", "fp32", "int8", "e4m3"])
def test_sparse24(golden, tag):
    d = golden("sparse")[f"s24_{tag}"]
    assert_bit_equal(orc.sparse24_mask(d["x"]), d["mask"], "2:4 keep mask")
    values, bitmask = orc.sparse24_compress(d["x"])
    assert_bit_equal(values, d["values"], "values")
    assert_bit_equal(bitmask, d["bitmask"], "bitmask")
    assert_bit_equal(orc.bitmask_decompress(values, bitmask, d["x"].shape), d["dense"], "dense")


def test_sparse24_all_weak_orderings(golden):
    d = golden("sparse")["s24_rank_patterns"]
    assert d["ranks"].shape[0] == 75
    assert_bit_equal(orc.sparse24_mask(d["ranks"].float()), d["mask"])
    assert_bit_equal(orc.sparse24_mask(d["ranks"]), d["mask_int8"])
    assert_bit_equal(orc.sparse24_mask(d["ranks"].to(torch.bfloat16)), d["mask_bf16"])
    # the mask is a function of the ordering only
    assert_bit_equal(d["mask"], d["mask_int8"]), assert_bit_equal(d["mask"], d["mask_bf16"])


def test_hadamard(golden):
    g = golden("hadamard")
    for n in (16, 64, 128, 256):
        H = g[f"det_{n}"]["H"]
        i = torch.arange(n)
        syl = 1 - 2 * (torch.tensor([[bin(int(a & b)).count("1") & 1 for b in i] for a in i]))
        assert torch.equal(H.long(), syl), n
    for name, d in g.items():
        if not (name.startswith("hadamard_") or name.startswith("random_")):
            continue
        m = d["matrix"]
        n = m.shape[0]
        signs = m[:, 0].clone()  # diag(Q) @ H: column 0 of H is all ones
        i = torch.arange(n)
        syl = 1 - 2 * (torch.tensor([[bin(int(a & b)).count("1") & 1 for b in i] for a in i]))
        assert torch.equal(m.long(), signs.long()[:, None] * syl), name
        side = 0 if "weight_input" in name else 1
        out = orc.hadamard(d["w"], n, signs=signs, inverse="_inv_" in name, side=side)
        if d["w"].dtype == torch.bfloat16:
            assert_bit_equal(out, d["out"], name)
        else:
            torch.testing.assert_close(out, d["out"], rtol=1e-6, atol=1e-7, msg=name)


def test_hadamard_whole_dimension(golden):
    """transforms as wide as the dimension (n = 1024, 2048; no head_dim), float64 offline path: bit-exact"""
    for name, d in golden("hadamard_full").items():
        n = int(name.rsplit("_", 1)[1])
        side = 0 if "weight_input" in name else 1
        out = orc.hadamard(d["w"], n, signs=d["signs"], inverse="_inv_" in name, side=side)
        assert_bit_equal(out, d["out"], name)


def test_mxfp4_scale_helpers_every_input(golden):
    """mxfp4_utils.py on all 65536 bf16 bit patterns and all 256 exponent bytes"""
    d = golden("mxfp4")
    x = torch.arange(65536, dtype=torch.int32).to(torch.uint16).view(torch.bfloat16)
    assert torch.equal(orc.mxfp4_round_pow2(x).view(torch.uint16), d["all_bf16"]["round_pow2_bits"])
    assert torch.equal(orc.mxfp4_generate_scales(x), d["all_bf16"]["scales"])
    e = torch.arange(256, dtype=torch.int32).to(torch.uint8)
    for key, dt in (("bf16", torch.bfloat16), ("f16", torch.float16), ("f32", torch.float32)):
        assert_bit_equal(orc.mxfp4_convert_scales(e, dt), d["all_exponents"][key], key)


def test_fp4_pack_every_16bit_input(golden):
    """pack_fp4_to_uint8 on all 65536 bf16 and f16 bit patterns and a float32 sweep; unpack on every byte"""
    d = golden("fp4_pack_all")
    bits = torch.arange(65536, dtype=torch.int32).to(torch.uint16).reshape(256, 256)
    assert torch.equal(orc.pack_fp4(bits.view(torch.bfloat16)), d["bf16_packed"])
    assert torch.equal(orc.pack_fp4(bits.view(torch.float16)), d["f16_packed"])
    assert torch.equal(orc.pack_fp4(d["f32"]), d["f32_packed"])
    every_byte = torch.arange(256, dtype=torch.int32).to(torch.uint8).reshape(16, 16)
    for key, dt in (("bf16", torch.bfloat16), ("f16", torch.float16), ("f32", torch.float32)):
        assert_bit_equal(orc.unpack_fp4(every_byte, 16, 32, dtype=dt), d["unpacked_" + key], key)


def test_marlin24_steps(golden):
    """CUTLASS 2:4 compaction + reordered meta, tile permutation + packing, scale permutation (marlin_24.py:124-273)"""
    for name, d in golden("marlin24").items():
        if name.startswith("permutations_"):
            continue
        bits, group = int(d["bits"]), int(d["group"])
        assert torch.equal(orc.cutlass24_decompress(d["sparse"], d["meta_reordered"]), d["dense_back"]), name
        sparse, meta = orc.cutlass24_compress(d["q"])
        assert torch.equal(sparse, d["sparse"]) and torch.equal(meta, d["meta_reordered"]), name
        assert torch.equal(orc.marlin24_pack_weight(sparse, bits), d["weight_packed"]), name
        grouped = group > 0 and group < sparse.shape[1]
        assert_bit_equal(orc.marlin24_pack_scales(d["scale"], grouped), d["scale_packed"], name)
        assert torch.equal(meta.reshape(meta.shape[1] // 2, meta.shape[0] * 2), d["meta"]), name



def test_generate_gparam_every_bf16_and_f16_maximum(golden):
    """`448 * 6 / amax` with the scalar on the left is amax.reciprocal() * 2688 in torch: two roundings in the min/max
    dtype.  Every positive finite bf16 and fp16 maximum and a float32 sample, against the reference's outputs."""
    g = golden("gparam_all")
    for tag in ("bf16", "f16", "f32"):
        mx, want = g[tag]["max"], g[tag]["global_scale"]
        zero = torch.zeros((), dtype=mx.dtype)
        got = torch.cat([orc.generate_gparam(zero, m) for m in mx])
        assert_bit_equal(got, want, f"global scale, {tag} maxima")
    mn, want = g["neg"]["min"], g["neg"]["global_scale"]
    got = torch.cat([orc.generate_gparam(m, -m / 2) for m in mn])
    assert_bit_equal(got, want, "global scale, dominated by the minimum")
