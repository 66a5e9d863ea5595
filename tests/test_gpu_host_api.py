"""The reference-facing Python API (same names and signatures as compressed-tensors) on the GPU,
against the reference's own outputs in tests/golden/."""
import pytest
import torch

from tests.helpers import assert_bit_equal

pytestmark = pytest.mark.gpu


def dev(t):
    return None if t is None else t.cuda()


def int_args(d, name):
    from compressed_tensors_b200.quantization import QuantizationArgs

    bits, sym, group = int(d["bits"]), bool(d["sym"]), int(d["group"])
    if "tensor" in name:
        return QuantizationArgs(num_bits=bits, symmetric=sym, strategy="tensor")
    if "channel" in name:
        return QuantizationArgs(num_bits=bits, symmetric=sym, strategy="channel")
    return QuantizationArgs(num_bits=bits, symmetric=sym, strategy="group", group_size=group)


@pytest.mark.parametrize("name", ["w4_sym_g128_bf16", "w4_asym_g128_bf16", "w8_sym_channel_bf16", "w8_asym_channel_bf16",
                                  "w4_sym_tensor_bf16", "w4_sym_g128_fp32", "w4_asym_g64_fp16", "w4_sym_channel_fp32"])
def test_quantize_dequantize_pack_compressor(golden, name):
    from compressed_tensors_b200.compressors import PackedQuantizationCompressor, pack_to_int32, unpack_from_int32
    from compressed_tensors_b200.quantization import calculate_qparams, dequantize, fake_quantize, quantize

    d = golden("int_quant")[name]
    args = int_args(d, name)
    x, scale, zp = dev(d["x"]), dev(d["scale"]), dev(d["zp"])
    s, z = calculate_qparams(dev(d["min"]), dev(d["max"]), args)
    assert_bit_equal(s.cpu(), d["scale"]), assert_bit_equal(z.cpu(), d["zp"])
    q8 = quantize(x, scale, zp, args, dtype=torch.int8)
    assert_bit_equal(q8.cpu(), d["q_int8"])
    assert_bit_equal(quantize(x, scale, zp, args).cpu(), d["q_float"], "dtype=None result dtype and values")
    assert_bit_equal(dequantize(q8, scale, zp, args).cpu(), d["dequant"])
    if "tensor" not in name:
        assert_bit_equal(dequantize(q8, scale, zp).cpu(), d["dequant_noargs"], "strategy inferred from the scale shape")
    assert_bit_equal(fake_quantize(x, scale, zp, args).cpu(), d["fake"])
    assert_bit_equal(pack_to_int32(q8, args.num_bits).cpu(), d["packed"])
    assert_bit_equal(unpack_from_int32(dev(d["packed"]), args.num_bits, x.shape).cpu(), d["unpacked"])
    comp = PackedQuantizationCompressor()
    cd = comp.compress_weight(x, scale, args, zero_point=zp)
    assert_bit_equal(cd["weight_packed"].cpu(), d["c_weight_packed"])
    assert cd["weight_shape"].dtype == torch.int64 and cd["weight_shape"].tolist() == list(x.shape)
    if "c_weight_zero_point" in d:
        assert_bit_equal(cd["weight_zero_point"].cpu(), d["c_weight_zero_point"])
    cd["weight_scale"] = scale
    assert_bit_equal(comp.decompress_weight(cd, args).cpu(), d["decompressed"])
    with pytest.raises(ValueError, match="global_scale is not supported"):
        comp.compress_weight(x, scale, args, zero_point=zp, global_scale=torch.ones(1))


def test_actorder(golden):
    from compressed_tensors_b200.quantization import QuantizationArgs, dequantize, fake_quantize, quantize

    d = golden("int_quant")["w4_sym_g64_actorder"]
    args = QuantizationArgs(num_bits=4, symmetric=True, strategy="group", group_size=64, actorder="group")
    x, scale, zp, g_idx = dev(d["x"]), dev(d["scale"]), dev(d["zp"]), dev(d["g_idx"])
    q8 = quantize(x, scale, zp, args, dtype=torch.int8, g_idx=g_idx)
    assert_bit_equal(q8.cpu(), d["q_int8"])
    assert_bit_equal(dequantize(q8, scale, zp, args, g_idx=g_idx).cpu(), d["dequant"])
    assert_bit_equal(fake_quantize(x, scale, zp, args, g_idx=g_idx).cpu(), d["fake"])
    # g_idx of all -1 means "column order" (forward.py:286)
    q_plain = quantize(x, scale, zp, args, dtype=torch.int8, g_idx=torch.full_like(g_idx, -1))
    assert_bit_equal(q_plain.cpu(), quantize(x, scale, zp, args, dtype=torch.int8).cpu())
    # the same tensor filled in afterwards (in place) is a new state: the remembered answer must not stick
    late = torch.full_like(g_idx, -1)
    quantize(x, scale, zp, args, dtype=torch.int8, g_idx=late)
    late.copy_(g_idx)
    assert_bit_equal(quantize(x, scale, zp, args, dtype=torch.int8, g_idx=late).cpu(), d["q_int8"])


def test_actorder_inside_graph_capture(golden):
    """Nothing may be read back to the host while a CUDA graph is captured: whether the column map is in use
    (forward.py:286) is then decided on the device."""
    from compressed_tensors_b200.quantization import QuantizationArgs, fake_quantize

    d = golden("int_quant")["w4_sym_g64_actorder"]
    args = QuantizationArgs(num_bits=4, symmetric=True, strategy="group", group_size=64, actorder="group")
    x, scale, zp, g_idx = dev(d["x"]), dev(d["scale"]), dev(d["zp"]), dev(d["g_idx"])
    unset = torch.full_like(g_idx, -1)
    plain = fake_quantize(x, scale, zp, args)
    fake_quantize(x, scale, zp, args, g_idx=g_idx)  # warm-up outside the capture
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            mapped = fake_quantize(x, scale, zp, args, g_idx=g_idx)
            ignored = fake_quantize(x, scale, zp, args, g_idx=unset)
    graph.replay()
    torch.cuda.synchronize()
    assert_bit_equal(mapped.cpu(), d["fake"])
    assert_bit_equal(ignored.cpu(), plain.cpu())


def test_fp8_api(golden):
    from compressed_tensors_b200.compressors import BaseCompressor
    from compressed_tensors_b200.quantization import (QuantizationArgs, compute_dynamic_scales_and_zp, dequantize,
                                                      fake_quantize, quantize)

    g = golden("fp8_quant")
    args_c = QuantizationArgs(num_bits=8, type="float", symmetric=True, strategy="channel")
    args_tok = QuantizationArgs(num_bits=8, type="float", symmetric=True, strategy="token", dynamic=True)
    args_b = QuantizationArgs(num_bits=8, type="float", symmetric=True, strategy="block", block_structure=[16, 64])
    for tag in ("channel_bf16", "channel_bf16_f32scale", "channel_fp16", "channel_fp32"):
        d = g[tag]
        x, scale, zp = dev(d["x"]), dev(d["scale"]), dev(d["zp"])
        q = quantize(x, scale, zp, args_c, dtype=torch.float8_e4m3fn)
        assert_bit_equal(q.cpu(), d["q"], tag)
        assert_bit_equal(quantize(x, scale, zp, args_c).cpu(), d["q_float"], tag)
        assert_bit_equal(dequantize(q, scale, zp, args_c).cpu(), d["dequant"], tag)
        assert_bit_equal(dequantize(q, scale).cpu(), d["dequant_noargs"], tag)
        assert_bit_equal(fake_quantize(x, scale, zp, args_c).cpu(), d["fake"], tag)
        comp = BaseCompressor.load_from_registry("float-quantized")
        cd = comp.compress_weight(x, scale, args_c, zero_point=zp)
        assert_bit_equal(cd["weight"].cpu(), d["c_weight"], tag)
        cd["weight_scale"] = scale
        assert_bit_equal(comp.decompress_weight(cd, args_c).cpu(), d["decompressed"], tag)
    d = g["token_bf16"]
    x = dev(d["x"])
    scale, zp = compute_dynamic_scales_and_zp(x, args_tok, module=None)
    assert_bit_equal(scale.cpu(), d["scale"]), assert_bit_equal(zp.cpu(), d["zp"])
    assert_bit_equal(quantize(x, scale, zp, args_tok, dtype=torch.float8_e4m3fn).cpu(), d["q"])
    assert_bit_equal(fake_quantize(x, scale, zp, args_tok).cpu(), d["fake"])
    d2 = g["token_2d"]
    s2, z2 = compute_dynamic_scales_and_zp(dev(d2["x"]), args_tok, module=None)
    assert_bit_equal(s2.cpu(), d2["scale"], "2-D TOKEN input collapses to one scale")
    d = g["block_bf16"]
    x, scale, zp = dev(d["x"]), dev(d["scale"]), dev(d["zp"])
    q = quantize(x, scale, zp, args_b, dtype=torch.float8_e4m3fn)
    assert_bit_equal(q.cpu(), d["q"])
    assert_bit_equal(dequantize(q, scale, zp, args_b).cpu(), d["dequant"])
    with pytest.raises(ValueError, match="not divisible by block_height"):
        quantize(x[:30], scale, zp, args_b)


def test_nvfp4_api(golden):
    from compressed_tensors_b200.compressors import NVFP4PackedCompressor, pack_fp4_to_uint8, unpack_fp4_from_uint8
    from compressed_tensors_b200.quantization import (QuantizationArgs, calculate_qparams, compute_dynamic_scales_and_zp,
                                                      dequantize, fake_quantize, generate_gparam, quantize)

    args = QuantizationArgs(num_bits=4, type="float", symmetric=True, strategy="tensor_group", group_size=16)
    for tag in ("a", "b"):
        d = golden("nvfp4")[tag]
        x, scale, zp, gs = dev(d["x"]), dev(d["scale"]), dev(d["zp"]), dev(d["global_scale"])
        assert_bit_equal(generate_gparam(dev(d["min"]), dev(d["max"])).cpu(), d["global_scale"])
        s, z = calculate_qparams(dev(d["gmin"]), dev(d["gmax"]), args, global_scale=gs)
        assert_bit_equal(s.cpu(), d["scale"]), assert_bit_equal(z.cpu(), d["zp"])
        s, _ = compute_dynamic_scales_and_zp(x, args, module=None, global_scale=gs)
        assert_bit_equal(s.cpu(), d["scale"], "dynamic local scales")
        q = quantize(x, scale, zp, args, global_scale=gs)
        assert_bit_equal(q.cpu(), d["q"])
        packed = pack_fp4_to_uint8(q)
        assert_bit_equal(packed.cpu(), d["packed"])
        assert_bit_equal(unpack_fp4_from_uint8(packed, *x.shape).cpu(), d["unpacked"])
        assert_bit_equal(dequantize(dev(d["unpacked"]), scale, global_scale=gs, dtype=torch.bfloat16).cpu(), d["dequant"])
        assert_bit_equal(fake_quantize(x, scale, zp, args, global_scale=gs).cpu(), d["fake"])
        comp = NVFP4PackedCompressor()
        cd = comp.compress_weight(x, scale, gs, args, zero_point=zp)
        assert_bit_equal(cd["weight_packed"].cpu(), d["c_weight_packed"])
        out = comp.decompress_weight({"weight_packed": cd["weight_packed"], "weight_scale": scale, "weight_global_scale": gs}, args)
        assert_bit_equal(out.cpu(), d["decompressed"])
    with pytest.raises(ValueError, match="even number of columns"):
        pack_fp4_to_uint8(torch.zeros(2, 3, device="cuda"))


def test_sparse_api(golden):
    from compressed_tensors_b200.compressors import (BitmaskCompressor, BitmaskTensor, Sparse24BitMaskCompressor, Sparse24BitMaskTensor,
                                                     bitmask_compress, bitmask_decompress, get_24_bytemasks,
                                                     sparse24_bitmask_compress, sparse24_bitmask_decompress)
    from compressed_tensors_b200.utils import pack_bitmasks, unpack_bitmasks

    g = golden("sparse")
    for tag in ("bf16", "fp16", "fp32", "e4m3"):
        for cols in (64, 13):
            d = g[f"bitmask_{tag}_{cols}"]
            values, bitmask, row_offsets = bitmask_compress(dev(d["x"]))
            assert_bit_equal(values.cpu(), d["values"]), assert_bit_equal(bitmask.cpu(), d["bitmask"])
            assert_bit_equal(row_offsets.cpu(), d["row_offsets"])
            assert_bit_equal(bitmask_decompress(values, bitmask, d["x"].shape).cpu(), d["dense"])
            assert_bit_equal(pack_bitmasks(unpack_bitmasks(bitmask, list(d["x"].shape))).cpu(), d["bitmask"])
    # compressor round trip from a CPU tensor, results on the CPU like the reference
    d = g["bitmask_bf16_64"]
    comp = BitmaskCompressor()
    sd = comp.compress({"layer.weight": d["x"]})
    assert set(sd) == {"layer.shape", "layer.compressed", "layer.bitmask", "layer.row_offsets"}
    assert all(not v.is_cuda for v in sd.values())
    assert_bit_equal(sd["layer.compressed"], d["values"])
    (name, dense), = list(comp.decompress(sd))
    assert name == "layer.weight"
    assert_bit_equal(dense.cpu(), d["dense"])
    assert BitmaskTensor.from_dense(d["x"]).curr_memory_size_bytes() == sum(v.numel() * v.element_size() for k, v in sd.items() if "shape" not in k)
    for tag in ("bf16", "fp32", "int8", "e4m3"):
        d = g[f"s24_{tag}"]
        assert_bit_equal(get_24_bytemasks(dev(d["x"])).cpu(), d["mask"])
        values, bitmask = sparse24_bitmask_compress(dev(d["x"]))
        assert_bit_equal(values.cpu(), d["values"]), assert_bit_equal(bitmask.cpu(), d["bitmask"])
        assert_bit_equal(sparse24_bitmask_decompress(values, bitmask, d["x"].shape).cpu(), d["dense"])
    d = g["s24_bf16"]
    comp = Sparse24BitMaskCompressor()
    sd = comp.compress({"m.weight": d["x"]})
    assert set(sd) == {"m.shape", "m.compressed", "m.bitmask"} and tuple(sd["m.shape"].shape) == (2, 1)
    (name, dense), = list(comp.decompress(sd))
    assert name == "m.weight"
    assert_bit_equal(dense.cpu(), d["dense"])
    with pytest.raises(ValueError, match="multiple of 4"):
        get_24_bytemasks(torch.zeros(3, 3, device="cuda"))
    meta_v, meta_b = sparse24_bitmask_compress(torch.empty(8, 16, device="meta"))
    assert meta_v.shape == (8, 8) and meta_b.shape == (8, 2)
    assert Sparse24BitMaskTensor.from_dense(d["x"]).curr_memory_size_bytes() > 0


def test_transform_factories(golden):
    from compressed_tensors_b200.transform import (HadamardFactory, RandomHadamardFactory, TransformArgs, TransformConfig, TransformScheme,
                                                   apply_transform_config)

    g = golden("hadamard")
    for tag, fac_cls, seed in (("hadamard", HadamardFactory, None), ("random", RandomHadamardFactory, 7)):
        for location in ("weight_input", "weight_output"):
            for inverse in (False, True):
                name = f"{tag}_{location}_{'inv' if inverse else 'fwd'}_bfloat16"
                d = g[name]
                o, i = d["w"].shape
                lin = torch.nn.Linear(i, o, bias=False, dtype=torch.bfloat16, device="cuda")
                lin.weight.data = dev(d["w"])
                scheme = TransformScheme(type=tag if tag == "hadamard" else "random-hadamard", head_dim=128,
                                         apply=[TransformArgs(targets=["Linear"], location=location, inverse=inverse)])
                fac = fac_cls("t", scheme, seed=seed)
                tr = fac.create_transform(lin, scheme.apply[0])
                assert torch.equal(tr.weight.data.to(torch.int8), d["matrix"]), name
                assert_bit_equal(tr(lin.weight.data).cpu(), d["out"], name)
    # config-level entry point, seed 7, fused into the weight
    d = g["random_weight_input_fwd_bfloat16"]
    model = torch.nn.Sequential(torch.nn.Linear(256, 16, bias=False, dtype=torch.bfloat16, device="cuda"))
    model[0].weight.data = dev(d["w"])
    cfg = TransformConfig(config_groups={"r": TransformScheme(type="random-hadamard", head_dim=128,
                                                              apply=[TransformArgs(targets=["Linear"], location="weight_input")])})
    apply_transform_config(model, cfg, seed=7)
    assert_bit_equal(model[0].weight.data.cpu(), d["out"])


def test_model_compressor_round_trip():
    """compress == compress_model, decompress_model restores fake-quantized weights, on a toy model."""
    from compressed_tensors_b200.compressors import ModelCompressor
    from compressed_tensors_b200.quantization import (QuantizationConfig, apply_quantization_config, calibrate_weight_qparams,
                                                      fake_quantize)

    torch.manual_seed(0)
    model = torch.nn.Sequential(torch.nn.Linear(256, 128, bias=False), torch.nn.ReLU(), torch.nn.Linear(128, 32, bias=True))
    model = model.to(torch.bfloat16).cuda()
    cfg = QuantizationConfig(config_groups={"W4A16": ["Linear"]}, format="pack-quantized")
    apply_quantization_config(model, cfg)
    expect = {}
    for name, m in model.named_modules():
        if isinstance(m, torch.nn.Linear):
            calibrate_weight_qparams(m)
            expect[name] = fake_quantize(m.weight.data, m.weight_scale.data, m.weight_zero_point.data, m.quantization_scheme.weights).cpu()
    mc = ModelCompressor(quantization_config=cfg)
    sd = mc.compress(model)
    assert "0.weight_packed" in sd and "0.weight_shape" in sd and "0.weight_scale" in sd and "0.weight" not in sd
    assert "0.weight_zero_point" not in sd, "symmetric zero points are dropped"
    assert "2.bias" in sd and all(not v.is_cuda for v in sd.values())
    assert sd["0.weight_packed"].dtype == torch.int32 and tuple(sd["0.weight_packed"].shape) == (128, 32)
    mc.compress_model(model)
    assert not hasattr(model[0], "weight")
    for k in ("0.weight_packed", "0.weight_scale", "2.weight_packed", "2.bias"):
        assert_bit_equal(dict(model.state_dict())[k].cpu(), sd[k], k)
    mc.decompress_model(model)
    for name, want in expect.items():
        got = dict(model.named_modules())[name].weight.data.cpu()
        assert got.dtype == want.dtype and torch.equal(got, want), name  # numeric equality, as the reference's reload test
    y = model(torch.randn(2, 256, dtype=torch.bfloat16, device="cuda"))
    assert y.shape == (2, 32)


@pytest.mark.parametrize("fmt,group", [("pack-quantized", "W4A16"), ("nvfp4-pack-quantized", "NVFP4A16"), ("float-quantized", "FP8")])
def test_disk_decompress_and_compressed_linear(tmp_path, fmt, group):
    """checkpoint on disk -> packed tensors opened on the GPU -> unpack + dequantize (quantized base.py:190-237), and
    CompressedLinear decompressing at its first forward (linear/compressed_linear.py:98-109): both give the bits of
    the in-memory decompress"""
    from safetensors.torch import save_file

    from compressed_tensors_b200.compressors import BaseCompressor, ModelCompressor
    from compressed_tensors_b200.linear import CompressedLinear
    from compressed_tensors_b200.quantization import (QuantizationConfig, QuantizationStatus, apply_quantization_config,
                                                      calibrate_weight_qparams)

    torch.manual_seed(1)
    model = torch.nn.Sequential(torch.nn.Linear(256, 128, bias=False), torch.nn.Linear(128, 64, bias=True)).to(torch.bfloat16).cuda()
    cfg = QuantizationConfig(config_groups={group: ["Linear"]}, format=fmt)
    apply_quantization_config(model, cfg)
    schemes = {}
    for name, m in model.named_modules():
        if isinstance(m, torch.nn.Linear):
            calibrate_weight_qparams(m)
            schemes[name] = m.quantization_scheme
    sd = ModelCompressor(quantization_config=cfg).compress(model)
    comp = BaseCompressor.load_from_registry(fmt)
    in_memory = {path: data["weight"] for path, data in comp.decompress(sd, names_to_scheme=schemes)}
    assert set(in_memory) == {"0", "1"}

    single = tmp_path / "model.safetensors"
    save_file({k: v.contiguous() for k, v in sd.items()}, str(single))
    for where in (str(single), str(tmp_path)):
        for device in ("cpu", "cuda:0"):
            from_disk = dict(comp.decompress(where, names_to_scheme=schemes, device=device))
            assert set(from_disk) == {"0", "1"}
            for path, data in from_disk.items():
                assert data["weight"].device.type == device.split(":")[0]
                assert_bit_equal(data["weight"].cpu(), in_memory[path].cpu(), f"{where} {path}")

    lin = torch.nn.Linear(256, 128, bias=False, dtype=torch.bfloat16).cuda()
    mod = CompressedLinear.from_linear(lin, schemes["0"], fmt)
    missing, unexpected = mod.load_state_dict({k.removeprefix("0."): v for k, v in sd.items() if k.startswith("0.")}, strict=False)
    assert not unexpected
    if fmt != "float-quantized":  # the naive formats keep their codes under the name `weight`
        assert not hasattr(mod, "weight")
    x = torch.randn(4, 256, dtype=torch.bfloat16, device="cuda")
    y = mod(x)
    assert mod.quantization_status == QuantizationStatus.FROZEN
    assert_bit_equal(mod.weight.data.cpu(), in_memory["0"].cpu(), "weight decompressed at the first forward")
    # the forward installed by initialize_module_for_quantization fake-quantizes the input where the scheme has input
    # activations (forward.py:355-412), as the reference's CompressedLinear does
    from compressed_tensors_b200.quantization import forward_quantize
    acts = schemes["0"].input_activations
    xin = x if acts is None else forward_quantize(mod, x, "input", acts)
    assert_bit_equal(y.cpu(), torch.nn.functional.linear(xin, in_memory["0"].cuda()).cpu(), "forward")
    assert_bit_equal(mod(x).cpu(), y.cpu(), "second forward reuses the dense weight (fake-quantizing it again changes nothing)")
    assert_bit_equal(mod.weight.data.cpu(), in_memory["0"].cpu(), "the dense weight is left as decompressed")


def test_hadamard_whole_dimension(golden):
    """HadamardFactory / RandomHadamardFactory without head_dim: the transform spans the whole input (weight_input) or
    output (weight_output) dimension, n = 1024 and 2048; float64 offline path, bit-exact against the reference; the
    fp32 mode of the same kernels within one bf16 step of the value"""
    from compressed_tensors_b200 import ops
    from compressed_tensors_b200.transform import TransformArgs, TransformFactory, TransformScheme

    for name, d in golden("hadamard_full").items():
        tag, rest = name.split("_", 1)
        location, direction, n = rest.rsplit("_", 2)
        n, inverse = int(n), direction == "inv"
        o, i = d["w"].shape
        lin = torch.nn.Linear(i, o, bias=False, dtype=torch.bfloat16, device="cuda")
        lin.weight.data = d["w"].cuda()
        scheme = TransformScheme(type="hadamard" if tag == "hadamard" else "random-hadamard",
                                 apply=[TransformArgs(targets=["Linear"], location=location, inverse=inverse)])
        fac = TransformFactory.from_scheme(scheme, name="t", seed=None if tag == "hadamard" else 7)
        tr = fac.create_transform(lin, scheme.apply[0])
        assert tr.weight.shape == (n, n) and torch.equal(tr.weight.data[:, 0].to(torch.int8).cpu(), d["signs"]), name
        assert_bit_equal(tr(lin.weight.data).cpu(), d["out"], name)
        fast = ops.hadamard(d["w"].cuda(), n, signs=d["signs"].cuda(), inverse=inverse, side=0 if location == "weight_input" else 1,
                            precision=torch.float32)
        want = d["out"].float()
        assert bool(((fast.cpu().float() - want).abs() <= want.abs() * 2.0 ** -7 + 1e-6).all()), name + " float32 mode"


def test_online_hadamard_hooks(golden):
    """input / output transforms on activations (transform/factory/base.py:132-167): the reference computes them
    as an fp32 matmul, the butterfly sums in another order, so the match is to one bf16 step / 1e-5 relative"""
    from compressed_tensors_b200.transform import TransformArgs, TransformFactory, TransformScheme
    from tests.helpers import bf16_ulp_distance

    g = golden("hadamard_online")
    for name, d in g.items():
        tag, location, direction, dtype = name.split("_")
        inverse = direction == "inv"
        i, o = (256, 16) if location == "input" else (16, 256)
        lin = torch.nn.Linear(i, o, bias=False, dtype=d["x"].dtype).cuda()
        scheme = TransformScheme(type="hadamard" if tag == "hadamard" else "random-hadamard", head_dim=128,
                                 apply=[TransformArgs(targets=["Linear"], location=location, inverse=inverse)])
        fac = TransformFactory.from_scheme(scheme, name="t", seed=None if tag == "hadamard" else 7)
        tr = fac.create_transform(lin, scheme.apply[0])
        assert torch.equal(tr.weight.data.to(torch.int8).cpu(), d["matrix"]), name
        y = tr(d["x"].cuda()).cpu()
        assert y.dtype == d["out"].dtype and y.shape == d["out"].shape
        if y.dtype == torch.bfloat16:
            assert bf16_ulp_distance(y, d["out"]) <= 1, name
        else:
            torch.testing.assert_close(y, d["out"], rtol=1e-5, atol=1e-6)
    # the hooks: a pre-hook rotates the input, a forward hook rotates the output
    torch.manual_seed(3)
    lin = torch.nn.Linear(256, 256, bias=False, dtype=torch.bfloat16).cuda()
    plain = torch.nn.Linear(256, 256, bias=False, dtype=torch.bfloat16).cuda()
    plain.weight.data.copy_(lin.weight.data)
    scheme = TransformScheme(type="hadamard", head_dim=128, apply=[TransformArgs(targets=["Linear"], location="input"),
                                                                   TransformArgs(targets=["Linear"], location="output", inverse=True)])
    fac = TransformFactory.from_scheme(scheme, name="R")
    fac.apply_to_model(torch.nn.Sequential(lin))
    assert {n for n, _ in lin.named_children()} == {"R_input", "R_output"}
    x = torch.randn(5, 256, dtype=torch.bfloat16, device="cuda")
    tin, tout = lin.R_input, lin.R_output
    assert_bit_equal(lin(x).cpu(), tout(plain(tin(x))).cpu(), "hooked forward")


def test_marlin24_compressor(golden):
    """Marlin24Compressor.compress and its steps against the reference's tensors (marlin_24.py:124-273)"""
    from compressed_tensors_b200 import ops
    from compressed_tensors_b200.compressors import BaseCompressor, Marlin24Compressor, compress_weight_24, pack_scales_24, pack_weight_24
    from compressed_tensors_b200.quantization import QuantizationArgs, QuantizationScheme

    comp = BaseCompressor.load_from_registry("marlin-24")
    assert isinstance(comp, Marlin24Compressor) and comp.compression_param_names == ("weight_packed", "scale_packed", "meta")
    from compressed_tensors_b200.utils import sparse_semi_structured_from_dense_cutlass, sparse_semi_structured_to_dense_cutlass

    for name, d in golden("marlin24").items():
        if name.startswith("permutations_"):
            continue
        bits, group = int(d["bits"]), int(d["group"])
        # the inverse conversion (semi_structured_conversions.py:216) on codes and on the 16-bit tensor
        assert_bit_equal(ops.cutlass24_decompress(d["sparse"].cuda(), d["meta_reordered"].cuda()).cpu(), d["dense_back"], name)
        s_h, m_h = sparse_semi_structured_from_dense_cutlass(d["q"].to(torch.float16))
        assert_bit_equal(sparse_semi_structured_to_dense_cutlass(s_h, m_h).cpu(), d["dense_back"].to(torch.float16), name)
        args = QuantizationArgs(num_bits=bits, symmetric=True, strategy="group" if group else "channel", group_size=group or None)
        # the steps on the reference's intermediate tensors
        sparse, meta = ops.cutlass24_compress(d["q"].cuda())
        assert_bit_equal(sparse.cpu(), d["sparse"], name), assert_bit_equal(meta.cpu(), d["meta_reordered"], name)
        s16, m16 = compress_weight_24(d["q"].to(torch.float16))  # the 16-bit element path takes the same decisions
        assert_bit_equal(s16.cpu(), d["sparse"].to(torch.float16), name), assert_bit_equal(m16.cpu(), d["meta_reordered"], name)
        unsigned = (d["sparse"].t().to(torch.int32) + (1 << bits) // 2).contiguous()
        assert_bit_equal(pack_weight_24(unsigned, args).cpu(), d["weight_packed"], name)
        scale_t = d["scale"].to(torch.float16).t().contiguous()
        assert_bit_equal(pack_scales_24(scale_t, args, unsigned.shape).cpu(), d["scale_packed"], name)
        # the whole compressor
        out = comp.compress({"l.weight": d["weight"].cuda(), "l.weight_scale": d["scale"].cuda(), "l.bias": torch.zeros(3)},
                            {"l": QuantizationScheme(targets=["Linear"], weights=args)})
        assert set(out) == {"l.weight_packed", "l.scale_packed", "l.meta", "l.bias"} and all(not v.is_cuda for v in out.values())
        for key in ("weight_packed", "scale_packed", "meta"):
            assert_bit_equal(out[f"l.{key}"], d[key], f"{name} {key}")
    dense = torch.ones(64, 64, dtype=torch.float16, device="cuda")
    with pytest.raises(ValueError, match="2:4 sparsity structure"):
        comp.compress({"l.weight": dense, "l.weight_scale": torch.ones(64, 1, device="cuda")},
                      {"l": QuantizationScheme(targets=["Linear"], weights=QuantizationArgs(num_bits=4, strategy="channel"))})
    with pytest.raises(ValueError, match="group size 128"):
        comp.validate_quant_compatability({"l": QuantizationScheme(targets=["Linear"], weights=QuantizationArgs(num_bits=4, strategy="group", group_size=64))})
    with pytest.raises(NotImplementedError):
        comp.decompress("x")


def test_randomized_hadamard(golden):
    """randomize=True (factory/hadamard.py:62, :104-108): same permutation as the reference for the same seed, and
    the permuted transform applied around the butterfly kernel gives the reference's bits (float64 offline) or its
    values to one bf16 step (fp32 online)"""
    from compressed_tensors_b200.transform import TransformArgs, TransformFactory, TransformScheme
    from tests.helpers import bf16_ulp_distance

    for name, d in golden("hadamard_randomize").items():
        tag, rest = name.split("_", 1)
        location, direction = rest.rsplit("_", 1)
        i, o = (16, 256) if location == "weight_output" else (256, 16)
        lin = torch.nn.Linear(i, o, bias=False, dtype=torch.bfloat16).cuda()
        scheme = TransformScheme(type="hadamard" if tag == "hadamard" else "random-hadamard", head_dim=128, randomize=True,
                                 apply=[TransformArgs(targets=["Linear"], location=location, inverse=direction == "inv")])
        tr = TransformFactory.from_scheme(scheme, name="t", seed=11).create_transform(lin, scheme.apply[0])
        assert torch.equal(tr.weight.data.to(torch.int8).cpu(), d["matrix"]) and torch.equal(tr.perm.data.cpu(), d["perm"]), name
        y = tr(d["x"].cuda()).cpu()
        if location == "input":
            assert bf16_ulp_distance(y, d["out"]) <= 1, name
        else:
            assert_bit_equal(y, d["out"], name)


def test_embedding_transforms(golden):
    """transforms fused into an Embedding weight (transform/utils/matrix.py:121-126), float64 offline: bit-exact"""
    from compressed_tensors_b200.transform import TransformArgs, TransformFactory, TransformScheme

    for name, d in golden("hadamard_embedding").items():
        tag, rest = name.split("_", 1)
        location, direction = rest.rsplit("_", 1)
        emb = torch.nn.Embedding(128, 128, dtype=torch.bfloat16).cuda()
        scheme = TransformScheme(type="random-hadamard", head_dim=128,
                                 apply=[TransformArgs(targets=["Embedding"], location=location, inverse=direction == "inv")])
        tr = TransformFactory.from_scheme(scheme, name="t", seed=7).create_transform(emb, scheme.apply[0])
        assert_bit_equal(tr(d["w"].cuda()).cpu(), d["out"], name)



def test_forward_quantize_and_wrapped_forward(golden):
    """forward_quantize (static group weights, dynamic per-token int8 / fp8 activations, static per-tensor input and
    output) and the quantized forward that initialize_module_for_quantization installs, against the reference's
    outputs: fake-quantized weights and inputs bit-exact; the layer output to the step that one bf16 unit of the
    matmul can move it by (the matmul itself is torch's, on another device than the reference's)"""
    from compressed_tensors_b200.quantization import (QuantizationArgs, QuantizationScheme, QuantizationStatus, disable_quantization,
                                                      enable_quantization, forward_quantize, initialize_module_for_quantization)

    cases = {
        "w4a16_g128": dict(weights=QuantizationArgs(num_bits=4, symmetric=True, strategy="group", group_size=128)),
        "w8a8_int_dynamic_token": dict(weights=QuantizationArgs(num_bits=8, symmetric=True, strategy="channel"),
                                       input_activations=QuantizationArgs(num_bits=8, symmetric=True, strategy="token", dynamic=True)),
        "w8a8_fp8_dynamic_token": dict(weights=QuantizationArgs(num_bits=8, type="float", symmetric=True, strategy="channel"),
                                       input_activations=QuantizationArgs(num_bits=8, type="float", symmetric=True, strategy="token", dynamic=True)),
        "w8a8_int_static_tensor_in_out": dict(weights=QuantizationArgs(num_bits=8, symmetric=False, strategy="channel"),
                                              input_activations=QuantizationArgs(num_bits=8, symmetric=True, strategy="tensor"),
                                              output_activations=QuantizationArgs(num_bits=8, symmetric=True, strategy="tensor")),
    }
    g = golden("forward_quantize")
    for name, sides in cases.items():
        d = g[name]
        scheme = QuantizationScheme(targets=["Linear"], **sides)
        lin = torch.nn.Linear(256, 128, bias=False, dtype=torch.bfloat16, device="cuda")
        lin.weight.data = d["w"].cuda()
        initialize_module_for_quantization(lin, scheme)
        for key in ("weight_scale", "weight_zero_point", "input_scale", "output_scale"):
            if key in d:
                assert getattr(lin, key).shape == d[key].shape and getattr(lin, key).dtype == d[key].dtype, f"{name} {key}"
                getattr(lin, key).data = d[key].cuda()
        lin.quantization_status = QuantizationStatus.FROZEN
        x = d["x"].cuda()
        assert_bit_equal(forward_quantize(lin, lin.weight.data, "weight", scheme.weights).cpu(), d["fq_weight"], name + " weight")
        if "fq_input" in d:
            assert_bit_equal(forward_quantize(lin, x, "input", scheme.input_activations).cpu(), d["fq_input"], name + " input")
        before = lin.weight.data.clone()
        y = lin(x).cpu().float()
        assert torch.equal(lin.weight.data, before), name + ": the weight is restored after the forward"
        want = d["y"].float()
        step = float(d["output_scale"].float().max()) if "output_scale" in d else 0.0
        assert bool(((y - want).abs() <= want.abs() * 2.0 ** -6 + 1e-3 + step).all()), name + " output"
        disable_quantization(lin)
        plain = torch.nn.functional.linear(x, lin.weight.data)
        assert torch.equal(lin(x), plain), name + ": disabled quantization is the plain layer"
        torch.testing.assert_close(lin(x).cpu().float(), d["y_disabled"].float(), rtol=2.0 ** -6, atol=1e-3)
        enable_quantization(lin)
        lin.quantization_status = QuantizationStatus.COMPRESSED  # the stored weight is taken as already quantized
        stored = lin.weight.data
        assert forward_quantize(lin, stored, "weight", scheme.weights) is stored


def test_mask_creator_and_structure_check():
    """mask_creator (semi_structured_conversions.py:313) keeps the two largest magnitudes of every run of four;
    tensor_follows_mask_structure (utils/helpers.py:93) accepts the pruned tensor and rejects the dense one"""
    from compressed_tensors_b200.utils import mask_creator, tensor_follows_mask_structure

    g = torch.Generator().manual_seed(8)
    w = torch.randn(64, 256, generator=g).to(torch.bfloat16)  # distinct magnitudes almost surely: no tie order involved
    mask = mask_creator(w.cuda())
    assert mask.dtype == torch.float32 and mask.shape == w.shape
    runs = w.float().abs().reshape(-1, 4)
    want = torch.ones_like(runs).scatter_(1, torch.argsort(runs, dim=1)[:, :2], 0.0).reshape(w.shape)
    ties = (runs.sort(dim=1).values.diff(dim=1) == 0).any(dim=1).reshape(-1, 1).expand(-1, 4).reshape(w.shape)
    assert torch.equal(mask.cpu()[~ties], want[~ties])
    assert bool((mask.reshape(-1, 4).sum(dim=1) == 2).all())
    assert tensor_follows_mask_structure((w.cuda() * mask.to(torch.bfloat16)))
    with pytest.raises(ValueError):
        tensor_follows_mask_structure(w.cuda() + 1.0)
