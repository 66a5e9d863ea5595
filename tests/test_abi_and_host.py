"""CPU-side checks: the C-ABI library loads and exports every symbol the header declares, schema
validation behaves like the reference's, the partitioner and the amax exchange work across ranks."""
import ctypes
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    from compressed_tensors_b200 import _build, _lib

    _build.build()
    header = open(os.path.join(ROOT, "include", "ctb200.h")).read()
    declared = set(re.findall(r"\b(ctb_[a-z0-9_]+)\s*\(", header))
    declared -= {"ctb_status", "ctb_dtype", "ctb_qtype", "ctb_codec", "ctb_qdesc"}
    assert len(declared) >= 24
    lib = ctypes.CDLL(_lib.LIB_PATH)
    for name in sorted(declared):
        assert hasattr(lib, name), f"{name} is declared in ctb200.h but not exported"
    lib.ctb_version.restype = ctypes.c_char_p
    assert b"sm_100a" in lib.ctb_version()
    assert ctypes.sizeof(_lib.QDesc) == 5 * 8 + 8 * 4


def test_no_cpu_fallback():
    from compressed_tensors_b200 import ops

    with pytest.raises(RuntimeError, match="no CPU fallback"):
        ops.pack_bitmasks(torch.zeros(2, 8, dtype=torch.bool))


def test_argument_errors_do_not_need_a_gpu():
    """Host-side validation mirrors the reference's exceptions; a null/invalid call returns a status, never traps."""
    from compressed_tensors_b200 import _lib as L

    lib = L.lib()
    assert lib.ctb_pack_int32(None, L.i64(1), L.i64(1), L.i64(1), L.i64(1), L.i32(4), None, None) == 4  # CTB_EINVAL_NULL
    d = L.QDesc(4, 10, 4, 1, 2, 0, 4, 0, 0, 4, 4, 0, 0)
    one = ctypes.c_void_p(16)  # never dereferenced: validation fails first
    assert lib.ctb_quantize(ctypes.byref(d), one, one, None, None, None, one, None) == 1  # cols % group
    assert b"divisble" in lib.ctb_last_error_string()
    d = L.QDesc(4, 8, 8, 1, 1, 1, 3, 0, 0, 4, 4, 0, 0)
    assert lib.ctb_quantize(ctypes.byref(d), one, one, None, None, None, one, None) == 7  # float with 3 bits
    assert lib.ctb_pack_fp4(one, L.i32(0), L.i64(2), L.i64(3), one, None) == 1
    assert lib.ctb_sparse24_mask(one, L.i32(0), L.i64(6), one, None) == 1
    assert lib.ctb_hadamard(one, L.i32(0), L.i64(4), L.i64(96), L.i32(96), None, L.i32(0), L.i32(0), L.i32(3), L.i32(1), one, None) == 7


def test_quantization_args_validation():
    from compressed_tensors_b200.quantization import QuantizationArgs, QuantizationStrategy, preset_name_to_scheme

    assert QuantizationArgs().strategy == QuantizationStrategy.TENSOR
    assert QuantizationArgs(group_size=128).strategy == QuantizationStrategy.GROUP
    assert QuantizationArgs(group_size=-1).strategy == QuantizationStrategy.CHANNEL
    assert QuantizationArgs(type="FLOAT").pytorch_dtype() == torch.float8_e4m3fn
    assert QuantizationArgs(num_bits=4).pytorch_dtype() == torch.int8
    with pytest.raises(ValueError):
        QuantizationArgs(strategy="token")  # static token quantization
    with pytest.raises(ValueError):
        QuantizationArgs(strategy="group")  # no group size
    with pytest.raises(ValueError):
        QuantizationArgs(strategy="channel", group_size=64)
    with pytest.raises(ValueError):
        QuantizationArgs(strategy="block")
    with pytest.raises(ValueError):
        QuantizationArgs(strategy="channel", actorder="group")
    with pytest.raises(ValueError):
        QuantizationArgs(bogus=1)
    assert QuantizationArgs(strategy="block", block_structure="128x128").block_structure == [128, 128]
    assert QuantizationArgs(strategy="token", dynamic=True).observer is None
    w4 = preset_name_to_scheme("w4a16", ["Linear"])
    assert w4.weights.num_bits == 4 and w4.weights.group_size == 128 and w4.weights.symmetric
    nv = preset_name_to_scheme("NVFP4", ["Linear"])
    assert nv.weights.strategy == QuantizationStrategy.TENSOR_GROUP and nv.input_activations.dynamic == "local"
    with pytest.raises(KeyError):
        preset_name_to_scheme("nope", [])


def test_registry():
    from compressed_tensors_b200.compressors import BaseCompressor, PackedQuantizationCompressor
    from compressed_tensors_b200.transform import HadamardFactory, TransformFactory

    assert isinstance(BaseCompressor.load_from_registry("pack-quantized"), PackedQuantizationCompressor)
    assert isinstance(BaseCompressor.load_from_registry("pack_quantized"), PackedQuantizationCompressor)
    assert TransformFactory.get_value_from_registry("hadamard") is HadamardFactory
    with pytest.raises(RuntimeError):
        BaseCompressor.register_value(dict, name="pack-quantized")  # same name, different class
    with pytest.raises(KeyError):
        BaseCompressor.get_value_from_registry("no-such-format")
    names = BaseCompressor.registered_names()
    for n in ("pack-quantized", "nvfp4-pack-quantized", "naive-quantized", "int-quantized", "float-quantized",
              "sparse-bitmask", "sparse-24-bitmask", "dense"):
        assert n in names


def test_hadamard_matrices(golden):
    from compressed_tensors_b200.transform import deterministic_hadamard_matrix, random_hadamard_matrix

    g = golden("hadamard")
    for n in (16, 64, 128, 256):
        assert torch.equal(deterministic_hadamard_matrix(n, torch.float64).to(torch.int8), g[f"det_{n}"]["H"])
        gen = torch.Generator().manual_seed(42)
        assert torch.equal(random_hadamard_matrix(n, torch.float64, gen=gen).to(torch.int8), g[f"rand_{n}_seed42"]["H"])
    with pytest.raises(ValueError):
        deterministic_hadamard_matrix(12)
    with pytest.raises(NotImplementedError):
        random_hadamard_matrix(32)


def test_partition_layers():
    from compressed_tensors_b200.parallel import LLAMA3_8B, linear_shapes, partition_layers

    for world in (1, 2, 3, 4, 8):
        parts = [list(partition_layers(32, world, r)) for r in range(world)]
        assert sorted(sum(parts, [])) == list(range(32))
        assert max(len(p) for p in parts) - min(len(p) for p in parts) <= 1
    assert sum(o * i for _, o, i in linear_shapes(LLAMA3_8B)) * 32 == 6979321856
    with pytest.raises(ValueError):
        partition_layers(32, 2, 2)


def _amax_worker(rank, world, port, out):
    import torch.distributed as dist

    from compressed_tensors_b200.parallel import allreduce_amax, partition_layers

    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    mn = torch.tensor(-1.0 - rank, dtype=torch.bfloat16)
    mx = torch.tensor(0.5 + 2 * rank, dtype=torch.bfloat16)
    gmn, gmx = allreduce_amax(mn, mx)
    layers = list(partition_layers(32, world, rank))
    got = [None] * world
    dist.all_gather_object(got, layers)
    if rank == 0:
        out.put((float(gmn), float(gmx), got, str(gmn.dtype)))
    dist.destroy_process_group()


def test_amax_exchange_two_ranks_gloo():
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + os.getpid() % 2000
    procs = [ctx.Process(target=_amax_worker, args=(r, 2, port, q)) for r in range(2)]
    [p.start() for p in procs]
    gmn, gmx, layers, dt = q.get(timeout=120)
    [p.join(60) for p in procs]
    assert all(p.exitcode == 0 for p in procs)
    assert (gmn, gmx) == (-2.0, 2.5) and dt == "torch.bfloat16"
    assert layers == [list(range(16)), list(range(16, 32))]


def test_safetensors_weight_mappings(tmp_path):
    """single file, folder with one file, sharded folder with an index: utils/safetensors_load.py:128-291"""
    import json

    from safetensors.torch import save_file

    from compressed_tensors_b200.utils import (get_nested_mappings_from_state_dict, get_nested_weight_mappings,
                                               get_safetensors_header, get_weight_mappings)

    a = {"m.0.weight_packed": torch.zeros(2, 2, dtype=torch.int32), "m.0.weight_scale": torch.ones(2, 1), "m.0.bias": torch.zeros(2)}
    b = {"m.1.weight_packed": torch.zeros(1, 2, dtype=torch.int32), "m.1.weight_shape": torch.tensor([1, 16])}
    one = tmp_path / "one.safetensors"
    save_file(a, str(one), metadata={"format": "pt"})
    assert set(get_safetensors_header(str(one))) == set(a) | {"__metadata__"}
    assert get_weight_mappings(str(one)) == {k: str(one) for k in a}
    folder = tmp_path / "single"
    folder.mkdir()
    save_file(a, str(folder / "model.safetensors"))
    assert get_weight_mappings(str(folder)) == {k: str(folder / "model.safetensors") for k in a}
    shard = tmp_path / "sharded"
    shard.mkdir()
    save_file(a, str(shard / "model-00001-of-00002.safetensors"))
    save_file(b, str(shard / "model-00002-of-00002.safetensors"))
    index = {"weight_map": {**{k: "model-00001-of-00002.safetensors" for k in a}, **{k: "model-00002-of-00002.safetensors" for k in b}}}
    (shard / "model.safetensors.index.json").write_text(json.dumps(index))
    nested, rest = get_nested_weight_mappings(str(shard), ("weight_packed", "weight_scale", "weight_shape"), return_unmatched_params=True)
    assert set(nested) == {"m.0", "m.1"} and set(nested["m.0"]) == {"weight_packed", "weight_scale"}
    assert nested["m.1"]["weight_shape"].endswith("model-00002-of-00002.safetensors") and set(rest) == {"m.0.bias"}
    assert set(get_nested_mappings_from_state_dict({**a, **b}, ("weight_packed",))) == {"m.0", "m.1"}
    with pytest.raises(ValueError):
        get_weight_mappings(str(tmp_path / "nothing-here"))


def test_initialize_qparams_shapes_and_compressed_linear_parameters():
    """lifecycle/initialize.py:153-277 shapes and dtypes; linear/compressed_linear.py:49-96 parameter set"""
    import warnings

    from compressed_tensors_b200.linear import CompressedLinear
    from compressed_tensors_b200.quantization import (QuantizationArgs, QuantizationScheme, QuantizationStatus,
                                                      initialize_module_for_quantization)

    def params(args, **kw):
        lin = torch.nn.Linear(256, 64, bias=False, dtype=torch.bfloat16)
        initialize_module_for_quantization(lin, QuantizationScheme(targets=["Linear"], weights=args), **kw)
        return {n: (tuple(p.shape), p.dtype) for n, p in lin.named_parameters() if n != "weight"}

    assert params(QuantizationArgs(num_bits=8, strategy="tensor")) == {
        "weight_scale": ((1,), torch.bfloat16), "weight_zero_point": ((1,), torch.int8)}
    assert params(QuantizationArgs(num_bits=8, strategy="channel"), force_zero_point=False) == {"weight_scale": ((64, 1), torch.bfloat16)}
    assert params(QuantizationArgs(num_bits=4, strategy="group", group_size=128, symmetric=False), force_zero_point=False) == {
        "weight_scale": ((64, 2), torch.bfloat16), "weight_zero_point": ((64, 2), torch.int8)}
    got = params(QuantizationArgs(num_bits=4, strategy="group", group_size=64, actorder="group"), force_zero_point=False)
    assert got["weight_g_idx"] == ((256,), torch.int32) and got["weight_scale"] == ((64, 4), torch.bfloat16)
    assert params(QuantizationArgs(num_bits=8, type="float", strategy="block", block_structure=[16, 64]), force_zero_point=False) == {
        "weight_scale": ((4, 4), torch.bfloat16)}
    got = params(QuantizationArgs(num_bits=4, type="float", strategy="tensor_group", group_size=16), force_zero_point=False)
    assert got == {"weight_global_scale": ((1,), torch.float32), "weight_scale": ((64, 16), torch.float8_e4m3fn)}

    lin = torch.nn.Linear(256, 64, bias=True, dtype=torch.bfloat16)
    scheme = QuantizationScheme(targets=["Linear"], weights=QuantizationArgs(num_bits=4, strategy="group", group_size=128))
    mod = CompressedLinear.from_linear(lin, scheme, "pack-quantized")
    assert isinstance(mod, CompressedLinear) and mod.quantization_status == QuantizationStatus.COMPRESSED
    assert {n: (tuple(p.shape), p.dtype) for n, p in mod.named_parameters()} == {
        "bias": ((64,), torch.bfloat16), "weight_scale": ((64, 2), torch.bfloat16),
        "weight_packed": ((64, 32), torch.int32), "weight_shape": ((2,), torch.int32)}
    with warnings.catch_warnings(record=True) as w:
        warnings.simplefilter("always")
        CompressedLinear(8, 8)
    assert any("from_linear" in str(x.message) for x in w)


def test_marlin24_permutation_tables(golden):
    """utils/permutations_24.py:32-65"""
    from compressed_tensors_b200.utils import get_permutations_24

    for bits in (4, 8):
        d = golden("marlin24")[f"permutations_{bits}"]
        perm, scale_perm, scale_perm_single = get_permutations_24(bits)
        assert torch.equal(perm.to(torch.int16), d["perm"])
        assert scale_perm == d["scale_perm"].tolist() and scale_perm_single == d["scale_perm_single"].tolist()
    with pytest.raises(ValueError):
        get_permutations_24(3)

