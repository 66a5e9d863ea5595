"""ModelCompressor against state dicts produced by the reference's own ModelCompressor
(tests/golden/model_compressor.pt, made by tests/golden/make_golden.py: gen_model_compressor): the calibrated
flow (rotation applied and scales present before compress), the fused flow (rotation and min-max calibration
inside the compress pass), host-resident and device-resident models, the stacked FP8 + 2:4 bitmask case, and
the checkpoint-on-disk decompress."""
import copy

import pytest
import torch

from tests.helpers import assert_bit_equal

pytestmark = pytest.mark.gpu

TOY = dict(layers=2, hidden=128, intermediate=256, kv=128, vocab=64)


def toy_llama(state, device="cpu", pin=False):
    """The module tree of the fixture generator, loaded with `state`."""
    from torch import nn

    def lin(o, i):
        return nn.Linear(i, o, bias=False, dtype=torch.bfloat16)

    class Attn(nn.Module):
        def __init__(self):
            super().__init__()
            self.q_proj, self.k_proj = lin(TOY["hidden"], TOY["hidden"]), lin(TOY["kv"], TOY["hidden"])
            self.v_proj, self.o_proj = lin(TOY["kv"], TOY["hidden"]), lin(TOY["hidden"], TOY["hidden"])

    class MLP(nn.Module):
        def __init__(self):
            super().__init__()
            self.gate_proj, self.up_proj = lin(TOY["intermediate"], TOY["hidden"]), lin(TOY["intermediate"], TOY["hidden"])
            self.down_proj = lin(TOY["hidden"], TOY["intermediate"])

    class Layer(nn.Module):
        def __init__(self):
            super().__init__()
            self.self_attn, self.mlp = Attn(), MLP()
            self.input_layernorm = nn.LayerNorm(TOY["hidden"], dtype=torch.bfloat16)

    class Inner(nn.Module):
        def __init__(self):
            super().__init__()
            self.layers = nn.ModuleList([Layer() for _ in range(TOY["layers"])])

    class Toy(nn.Module):
        def __init__(self):
            super().__init__()
            self.model = Inner()
            self.lm_head = lin(TOY["vocab"], TOY["hidden"])

    m = Toy()
    m.load_state_dict({k: v.clone() for k, v in state.items()})
    if device != "cpu":
        m = m.to(device)
    elif pin:
        for p in m.parameters():
            p.data = p.data.pin_memory()
    return m


def w4a16_configs():
    from compressed_tensors_b200.quantization import QuantizationArgs, QuantizationConfig, QuantizationScheme
    from compressed_tensors_b200.transform import TransformArgs, TransformConfig, TransformScheme

    tcfg = TransformConfig(config_groups={"u": TransformScheme(type="random-hadamard", head_dim=128, apply=[
        TransformArgs(targets=["Linear"], ignore=["lm_head"], location="weight_input")])})
    qcfg = QuantizationConfig(config_groups={"group_0": QuantizationScheme(
        targets=["Linear"], weights=QuantizationArgs(num_bits=4, symmetric=True, strategy="group", group_size=128))},
        ignore=["lm_head"], format="pack-quantized")
    return tcfg, qcfg


def fp8_sparse_configs():
    from compressed_tensors_b200.config import Sparse24BitMaskConfig
    from compressed_tensors_b200.quantization import QuantizationArgs, QuantizationConfig, QuantizationScheme

    qcfg = QuantizationConfig(config_groups={"group_0": QuantizationScheme(
        targets=["Linear"], weights=QuantizationArgs(num_bits=8, type="float", symmetric=True, strategy="channel"))},
        ignore=["lm_head"], format="float-quantized")
    scfg = Sparse24BitMaskConfig(targets=["Linear"], ignore=["lm_head"], sparsity_structure="2:4")
    return scfg, qcfg


def calibrate(model):
    from compressed_tensors_b200.quantization import calibrate_weight_qparams

    for m in model.modules():
        if getattr(m, "quantization_scheme", None) is not None and hasattr(m, "weight"):
            if m.weight.is_cuda:
                calibrate_weight_qparams(m)
            else:  # min-max calibration runs on the device; a host-resident model gets the parameters back
                w = m.weight.data
                m.weight.data = w.cuda()
                calibrate_weight_qparams(m)
                for name, p in list(m._parameters.items()):
                    if p is not None:
                        p.data = p.data.cpu()
                m.weight.data = w


def check_state(got, want, what):
    assert set(got.keys()) == set(want.keys()), f"{what}: keys differ: {sorted(set(got) ^ set(want))}"
    for k, v in want.items():
        assert_bit_equal(got[k].detach().cpu(), v, f"{what}: {k}")


@pytest.mark.parametrize("where", ["cuda", "cpu", "cpu-pinned"])
def test_calibrated_flow_matches_reference(golden, where):
    """apply_transform_config -> min-max scales -> ModelCompressor.compress / compress_model / decompress_model:
    every tensor of the reference's state dicts, bit for bit."""
    from compressed_tensors_b200.compressors import ModelCompressor
    from compressed_tensors_b200.quantization import apply_quantization_config
    from compressed_tensors_b200.transform import apply_transform_config

    g = golden("model_compressor")["w4a16_rot"]
    tcfg, qcfg = w4a16_configs()
    model = toy_llama(g["original"], device="cuda" if where == "cuda" else "cpu", pin=where == "cpu-pinned")
    if where == "cuda":
        apply_transform_config(model, tcfg)
    else:  # the stand-alone rotation runs on the device
        model.cuda()
        apply_transform_config(model, tcfg)
        model.cpu()
        if where == "cpu-pinned":
            for p in model.parameters():
                p.data = p.data.pin_memory()
    assert_bit_equal(model.model.layers[0].self_attn.q_proj.weight.data.cpu(), g["rotated_q_proj"], "rotated q_proj")
    apply_quantization_config(model, qcfg)
    calibrate(model)
    mc = ModelCompressor(quantization_config=copy.deepcopy(qcfg))
    sd = mc.compress(model)
    assert all(not v.is_cuda for v in sd.values()), "compress() returns host tensors"
    check_state(sd, g["compressed"], f"compress ({where})")
    assert hasattr(model.lm_head, "weight") and hasattr(model.model.layers[0].mlp.down_proj, "weight"), "compress() leaves the model alone"
    mc.compress_model(model)
    got = dict(model.state_dict())
    assert {k: (str(v.dtype), tuple(v.shape)) for k, v in got.items()} == g["inplace_keys"]
    check_state(got, g["compressed"], f"compress_model ({where})")
    dev = "cuda" if where == "cuda" else "cpu"
    assert all(v.device.type == dev for v in got.values()), "compressed parameters stay on the module's device"
    mc.decompress_model(model)
    got = dict(model.state_dict())
    assert {k: (str(v.dtype), tuple(v.shape)) for k, v in got.items()} == g["decompressed_keys"]
    for k, v in g["decompressed"].items():
        assert_bit_equal(got[k].cpu(), v, f"decompress_model ({where}): {k}")


@pytest.mark.parametrize("where", ["cuda", "cpu-pinned"])
@pytest.mark.parametrize("precision", ["exact", "tensor"])
def test_fused_flow_matches_reference(golden, where, precision):
    """transform_config handed to ModelCompressor and not yet applied, no scales on the model: the compress pass
    rotates, calibrates, quantizes and packs in one kernel.  float64 rotation: the reference's state dict bit for
    bit.  tcgen05 rotation: identical to the calibrated flow run on the tensor-core-rotated weights (the staged
    check), and the dequantized weights within the 1e-3 relative tolerance of the reference's."""
    from compressed_tensors_b200 import ops
    from compressed_tensors_b200.compressors import ModelCompressor
    from compressed_tensors_b200.quantization import apply_quantization_config

    g = golden("model_compressor")["w4a16_rot"]
    tcfg, qcfg = w4a16_configs()
    model = toy_llama(g["original"], device="cuda" if where == "cuda" else "cpu", pin=where != "cuda")
    apply_quantization_config(model, qcfg)
    mc = ModelCompressor(quantization_config=copy.deepcopy(qcfg), transform_config=tcfg, rotation_precision=precision)
    launches0 = mc.engine.launches
    mc.compress_model(model)
    assert mc.engine.launches - launches0 == 1, "every weight of the model goes through one launch"
    assert model.transform_config is tcfg, "the model is marked as transformed"
    got = dict(model.state_dict())
    assert set(got) == set(g["compressed"])
    if precision == "exact":
        check_state(got, g["compressed"], f"fused compress_model ({where})")
    else:
        signs = None
        for name, w in g["original"].items():
            if "layers" not in name or "layernorm" in name:
                continue
            prefix = name.removesuffix(".weight")
            if signs is None:
                from compressed_tensors_b200.transform.utils.hadamard import random_hadamard_signs
                signs = random_hadamard_signs(128, torch.Generator()).to(torch.int8).cuda()
            rot = ops.hadamard(w.cuda(), 128, signs=signs, precision=ops.ROT_TENSOR)
            words, scale = ops.absmax_quantize(rot, qtype=ops.QINT, bits=4, col_group=128, codec="pack32")
            assert_bit_equal(got[prefix + ".weight_packed"].cpu(), words.cpu(), f"staged {prefix}")
            assert_bit_equal(got[prefix + ".weight_scale"].cpu(), scale.cpu(), f"staged scale {prefix}")
    mc.decompress_model(model)
    got = dict(model.state_dict())
    for k, v in g["decompressed"].items():
        if precision == "exact":
            assert_bit_equal(got[k].cpu(), v, f"decompress after fused compress ({where}): {k}")
        else:
            rel = float((got[k].cpu().double() - v.double()).norm() / v.double().norm().clamp_min(1e-30))
            assert rel <= 0.1, (k, rel)  # int4 steps may flip where a rotated value moved by a rounding: bounded, not bit-equal


def test_fused_flow_state_dict_path_and_pipelined(golden):
    """compress() (state-dict path) with a pending transform, and compress_model + decompress_model inside
    `pipelined()`: the same bits as the synchronous calls."""
    from compressed_tensors_b200.compressors import ModelCompressor
    from compressed_tensors_b200.quantization import apply_quantization_config

    g = golden("model_compressor")["w4a16_rot"]
    tcfg, qcfg = w4a16_configs()
    model = toy_llama(g["original"], pin=True)
    apply_quantization_config(model, qcfg)
    mc = ModelCompressor(quantization_config=copy.deepcopy(qcfg), transform_config=tcfg)
    sd = mc.compress(model)
    check_state(sd, g["compressed"], "fused compress()")
    assert getattr(model, "transform_config", None) is None, "the model was not modified: the transform stays pending"
    with mc.pipelined():
        mc.compress_model(model)
        mc.decompress_model(model)
    got = dict(model.state_dict())
    for k, v in g["compressed"].items():
        assert_bit_equal(got[k].cpu(), v, f"pipelined: {k}")
    for k, v in g["decompressed"].items():
        assert_bit_equal(got[k].cpu(), v, f"pipelined decompress: {k}")
    assert all(v.device.type == "cpu" for v in got.values())


def test_reuse_buffers_cycles_equal_the_general_path(golden):
    """Three compress_model + decompress_model cycles with `reuse_buffers`: the second and third run as two launches
    over the first cycle's buffers and give the bits of a compressor that allocates afresh every time; a parameter
    replaced behind the compressor's back sends the next call down the general path."""
    from compressed_tensors_b200.compressors import ModelCompressor
    from compressed_tensors_b200.quantization import apply_quantization_config

    g = golden("model_compressor")["w4a16_rot"]
    tcfg, qcfg = w4a16_configs()
    models, mcs = [], []
    for reuse in (True, False):
        m = toy_llama(g["original"], device="cuda")
        apply_quantization_config(m, qcfg)
        models.append(m)
        mcs.append(ModelCompressor(quantization_config=copy.deepcopy(qcfg), transform_config=tcfg, reuse_buffers=reuse))
    for cycle in range(3):
        states = []
        for m, mc in zip(models, mcs):
            if getattr(m, "transform_config", None) is not None:
                del m.transform_config
            n0 = mc.engine.launches
            mc.compress_model(m)
            comp = {k: v.detach().cpu().clone() for k, v in m.state_dict().items()}
            mc.decompress_model(m)
            states.append((comp, {k: v.detach().cpu().clone() for k, v in m.state_dict().items()}, mc.engine.launches - n0))
        assert states[0][2] == 2 and states[1][2] == 2
        check_state(states[0][0], states[1][0], f"cycle {cycle} compressed")
        check_state(states[0][1], states[1][1], f"cycle {cycle} decompressed")
        if cycle == 0:
            check_state(states[0][0], g["compressed"], "first cycle against the reference")
    assert mcs[0]._cycle is not None and mcs[0]._cycle.ready
    lin = models[0].model.layers[0].mlp.down_proj
    lin.weight = torch.nn.Parameter(lin.weight.data.clone(), requires_grad=False)  # not the tensor the record knows
    del models[0].transform_config, models[1].transform_config
    mcs[0].compress_model(models[0])
    mcs[1].compress_model(models[1])
    check_state(dict(models[0].state_dict()), {k: v.cpu() for k, v in models[1].state_dict().items()}, "after a foreign parameter")


@pytest.mark.parametrize("where", ["cuda", "cpu"])
def test_stacked_fp8_and_sparse24_matches_reference(golden, where):
    """FP8 per-channel weights (float-quantized) stacked with sparse-24-bitmask through both configs."""
    from compressed_tensors_b200.compressors import ModelCompressor
    from compressed_tensors_b200.quantization import apply_quantization_config

    g = golden("model_compressor")["fp8_sparse24"]
    scfg, qcfg = fp8_sparse_configs()
    model = toy_llama(g["original"], device=where)
    apply_quantization_config(model, qcfg)
    calibrate(model)
    mc = ModelCompressor(sparsity_config=scfg, quantization_config=copy.deepcopy(qcfg))
    sd = mc.compress(model)
    check_state(sd, g["compressed"], f"stacked compress ({where})")
    mc.compress_model(model)
    got = dict(model.state_dict())
    assert {k: (str(v.dtype), tuple(v.shape)) for k, v in got.items()} == g["inplace_keys"]
    check_state(got, g["compressed"], f"stacked compress_model ({where})")
    mc.decompress_model(model)
    got = dict(model.state_dict())
    assert {k: (str(v.dtype), tuple(v.shape)) for k, v in got.items()} == g["decompressed_keys"]
    for k, v in g["decompressed"].items():
        assert_bit_equal(got[k].cpu(), v, f"stacked decompress_model ({where}): {k}")


@pytest.mark.parametrize("where", ["cuda", "cpu", "cpu-pinned"])
def test_fp8_channel_whole_shard_matches_reference(golden, where):
    """FP8 per-channel weights alone (float-quantized): every quantized weight goes through the whole-shard FP8 entry
    points, one launch per direction and device-resident call, and equals the reference's bit for bit."""
    from compressed_tensors_b200.compressors import ModelCompressor
    from compressed_tensors_b200.quantization import apply_quantization_config

    both = golden("model_compressor")
    g, original = both["fp8_channel"], both["fp8_sparse24"]["original"]
    _, qcfg = fp8_sparse_configs()
    model = toy_llama(original, device="cuda" if where == "cuda" else "cpu", pin=where == "cpu-pinned")
    apply_quantization_config(model, qcfg)
    calibrate(model)
    mc = ModelCompressor(quantization_config=copy.deepcopy(qcfg))
    sd = mc.compress(model)
    assert {k: (str(v.dtype), tuple(v.shape)) for k, v in sd.items()} == g["compressed_keys"]
    for k, v in g["compressed"].items():
        assert_bit_equal(sd[k].cpu(), v, f"compress ({where}): {k}")
    before = mc.engine.launches
    mc.compress_model(model)
    if where == "cuda":
        assert mc.engine.launches - before == 1, "one launch for every quantized weight of the model"
    got = dict(model.state_dict())
    assert {k: (str(v.dtype), tuple(v.shape)) for k, v in got.items()} == g["inplace_keys"]
    for k, v in g["compressed"].items():
        assert_bit_equal(got[k].cpu(), v, f"compress_model ({where}): {k}")
    before = mc.engine.launches
    mc.decompress_model(model)
    if where == "cuda":
        assert mc.engine.launches - before == 1
    got = dict(model.state_dict())
    assert {k: (str(v.dtype), tuple(v.shape)) for k, v in got.items()} == g["decompressed_keys"]
    for k, v in g["decompressed"].items():
        assert_bit_equal(got[k].cpu(), v, f"decompress_model ({where}): {k}")


@pytest.mark.parametrize("where", ["cuda", "cpu"])
def test_nvfp4_whole_shard_matches_reference(golden, where):
    """NVFP4 (nvfp4-pack-quantized: e2m1 codes, e4m3 group-16 scales under an fp32 global scale): every quantized
    weight goes through the whole-shard NVFP4 entry points and equals the reference's bit for bit."""
    from compressed_tensors_b200.compressors import ModelCompressor
    from compressed_tensors_b200.quantization import QuantizationArgs, QuantizationConfig, QuantizationScheme, apply_quantization_config

    both = golden("model_compressor")
    g, original = both["nvfp4"], both["fp8_sparse24"]["original"]
    qcfg = QuantizationConfig(config_groups={"group_0": QuantizationScheme(
        targets=["Linear"], weights=QuantizationArgs(num_bits=4, type="float", symmetric=True, strategy="tensor_group", group_size=16))},
        ignore=["lm_head"], format="nvfp4-pack-quantized")
    model = toy_llama(original, device=where)
    apply_quantization_config(model, qcfg)
    calibrate(model)
    mc = ModelCompressor(quantization_config=copy.deepcopy(qcfg))
    sd = mc.compress(model)
    assert {k: (str(v.dtype), tuple(v.shape)) for k, v in sd.items()} == g["compressed_keys"]
    for k, v in g["compressed"].items():
        assert_bit_equal(sd[k].cpu(), v, f"compress ({where}): {k}")
    before = mc.engine.launches
    mc.compress_model(model)
    if where == "cuda":
        assert mc.engine.launches - before == 1, "one launch for every quantized weight of the model"
    got = dict(model.state_dict())
    assert {k: (str(v.dtype), tuple(v.shape)) for k, v in got.items()} == g["inplace_keys"]
    for k, v in g["compressed"].items():
        assert_bit_equal(got[k].cpu(), v, f"compress_model ({where}): {k}")
    before = mc.engine.launches
    mc.decompress_model(model)
    if where == "cuda":
        assert mc.engine.launches - before == 1
    got = dict(model.state_dict())
    assert {k: (str(v.dtype), tuple(v.shape)) for k, v in got.items()} == g["decompressed_keys"]
    for k, v in g["decompressed"].items():
        assert_bit_equal(got[k].cpu(), v, f"decompress_model ({where}): {k}")


def test_decompress_from_disk(golden, tmp_path):
    """ModelCompressor.decompress(model_path, model): the reference's compressed state dict saved as safetensors,
    decompressed into a fresh dense model."""
    from safetensors.torch import save_file

    from compressed_tensors_b200.compressors import ModelCompressor

    g = golden("model_compressor")["w4a16_rot"]
    _, qcfg = w4a16_configs()
    save_file({k: v.contiguous() for k, v in g["compressed"].items()}, str(tmp_path / "model.safetensors"))
    for dev in ("cuda", "cpu"):
        model = toy_llama(g["original"], device=dev)
        ModelCompressor(quantization_config=copy.deepcopy(qcfg)).decompress(str(tmp_path), model)
        for k, v in g["decompressed"].items():
            got = dict(model.state_dict())[k]
            assert got.device.type == dev
            assert_bit_equal(got.cpu(), v, f"decompress from disk ({dev}): {k}")
        assert_bit_equal(model.model.layers[1].mlp.down_proj.weight_scale.data.cpu(),
                         g["compressed"]["model.layers.1.mlp.down_proj.weight_scale"], "scales are loaded with the weights")


def test_llama_layer_through_model_compressor_matches_oracle():
    """One full-size Llama-3-8B decoder layer (7 Linears, 218 M elements) through the fused compress pass and the
    batched decompress: float64 rotation bit-exact against the CPU oracle, tcgen05 rotation checked in stages.  This
    drives the multi-tensor table (one tensor map over all seven weights), not single-tensor calls."""
    from compressed_tensors_b200 import ops, parallel
    from compressed_tensors_b200.compressors import ModelCompressor
    from compressed_tensors_b200.quantization import apply_quantization_config
    from compressed_tensors_b200.transform.utils.hadamard import random_hadamard_signs
    from oracle import ref as orc

    tcfg, qcfg = w4a16_configs()
    shapes = parallel.linear_shapes(parallel.LLAMA3_8B)

    def build():
        layer = torch.nn.Module()
        g = torch.Generator().manual_seed(5)
        for name, o, i in shapes:
            parent = layer
            *path, leaf = name.split(".")
            for p in path:
                if not hasattr(parent, p):
                    parent.add_module(p, torch.nn.Module())
                parent = getattr(parent, p)
            lin = torch.nn.Linear(i, o, bias=False, dtype=torch.bfloat16, device="meta")
            lin.weight = torch.nn.Parameter((torch.randn(o, i, generator=g) * 0.02).to(torch.bfloat16).cuda(), requires_grad=False)
            parent.add_module(leaf, lin)
        apply_quantization_config(layer, qcfg)
        return layer

    signs = random_hadamard_signs(128, torch.Generator()).to(torch.int8)
    import os

    orc.set_threads(os.cpu_count() or 1)
    for precision in ("exact", "tensor"):
        layer = build()
        dense = {n: m.weight.data.clone() for n, m in layer.named_modules() if isinstance(m, torch.nn.Linear)}
        mc = ModelCompressor(quantization_config=copy.deepcopy(qcfg), transform_config=tcfg, rotation_precision=precision)
        mc.compress_model(layer)
        packed = {n: (m.weight_packed.data.cpu(), m.weight_scale.data.cpu()) for n, m in layer.named_modules() if hasattr(m, "weight_packed")}
        mc.decompress_model(layer)
        for name, o, i in shapes:
            w = dense[name]
            if precision == "exact":
                rot = orc.hadamard(w.cpu(), 128, signs=signs)
            else:
                rot = ops.hadamard(w, 128, signs=signs.cuda(), precision=ops.ROT_TENSOR).cpu()
                ref_rot = orc.hadamard(w.cpu(), 128, signs=signs)
                rel = float((rot.double() - ref_rot.double()).norm() / ref_rot.double().norm())
                assert rel <= 1e-3, (name, rel)
            mn, mx = orc.minmax(rot, 1, 128)
            scale, zp = orc.calculate_qparams(mn, mx, qtype=orc.QINT, bits=4, symmetric=True)
            kw = dict(qtype=orc.QINT, bits=4, col_group=128, row_group=1, scale_row_stride=i // 128)
            words = orc.pack_int32(orc.quantize(rot, scale, zp, out_dtype=torch.int8, **kw), 4)
            assert_bit_equal(packed[name][1], scale, f"{precision} {name} scale")
            assert_bit_equal(packed[name][0], words, f"{precision} {name} words")
            deq = orc.dequantize(orc.unpack_int32(words, 4, (o, i)), scale, None, out_dtype=torch.bfloat16, **kw)
            got = dict(layer.named_modules())[name].weight.data.cpu()
            assert_bit_equal(got, deq, f"{precision} {name} dequantized")
