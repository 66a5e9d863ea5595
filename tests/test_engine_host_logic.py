"""Host-side logic of the model loop that needs no GPU: which whole-shard entry point a module's job is given,
what a planned step will produce, how the column-order test of `g_idx` is remembered, how jobs are cut into steps."""
import torch

from compressed_tensors_b200.compressors.model_compressors import engine as E
from compressed_tensors_b200.compressors import BaseCompressor
from compressed_tensors_b200.quantization import QuantizationArgs, QuantizationScheme
from compressed_tensors_b200.quantization.lifecycle import forward as F


def _job(state, args, fmt, sparse=False, transforms=()):
    comp = BaseCompressor.load_from_registry(fmt)
    comp._format_name = fmt
    return E.Job("m", state, QuantizationScheme(targets=["Linear"], weights=args), comp, sparse, transforms)


W4 = QuantizationArgs(num_bits=4, symmetric=True, strategy="group", group_size=128)
F8 = QuantizationArgs(num_bits=8, type="float", symmetric=True, strategy="channel")
F4 = QuantizationArgs(num_bits=4, type="float", symmetric=True, strategy="tensor_group", group_size=16)


def test_compress_kinds():
    eng = E.CodecEngine()
    w = torch.zeros(256, 512, dtype=torch.bfloat16)
    j = _job({"weight": w, "weight_scale": torch.zeros(256, 4, dtype=torch.bfloat16)}, W4, "pack-quantized")
    eng.classify_compress(j)
    assert j.kind == "q4"
    j = _job({"weight": w, "weight_scale": torch.zeros(256, 4, dtype=torch.float32)}, W4, "pack-quantized")
    eng.classify_compress(j)
    assert j.kind == "generic", "fp32 scales go through the per-tensor compressor"
    j = _job({"weight": w, "weight_scale": torch.zeros(256, 4, dtype=torch.bfloat16), "weight_g_idx": torch.zeros(512, dtype=torch.int32)},
             W4, "pack-quantized")
    eng.classify_compress(j)
    assert j.kind == "generic"
    j = _job({"weight": w, "weight_scale": torch.zeros(256, 1, dtype=torch.bfloat16)}, F8, "float-quantized")
    eng.classify_compress(j)
    assert j.kind == "q8c"
    j = _job({"weight": w, "weight_scale": torch.zeros(256, 1, dtype=torch.bfloat16)}, F8, "float-quantized", sparse=True)
    eng.classify_compress(j)
    assert j.kind == "generic", "stacked with a sparsity compressor: the one-pass FP8 + 2:4 kernel, per module"
    j = _job({"weight": w, "weight_scale": torch.zeros(256, 32, dtype=torch.float8_e4m3fn),
              "weight_global_scale": torch.ones(1, dtype=torch.float32)}, F4, "nvfp4-pack-quantized")
    eng.classify_compress(j)
    assert j.kind == "q4f"
    j = _job({"weight": w, "weight_scale": torch.zeros(256, 32, dtype=torch.float8_e4m3fn)}, F4, "nvfp4-pack-quantized")
    eng.classify_compress(j)
    assert j.kind == "generic", "no global scale"
    j = _job({"weight": w.float(), "weight_scale": torch.zeros(256, 1, dtype=torch.bfloat16)}, F8, "float-quantized")
    eng.classify_compress(j)
    assert j.kind == "generic", "fp32 weights"


def test_decompress_kinds():
    eng = E.CodecEngine()
    j = _job({"weight_packed": torch.zeros(256, 64, dtype=torch.int32), "weight_scale": torch.zeros(256, 4, dtype=torch.bfloat16),
              "weight_shape": torch.tensor([256, 512])}, W4, "pack-quantized")
    eng.classify_decompress(j)
    assert (j.kind, j.shape) == ("dq4", (256, 512))
    j = _job({"weight": torch.zeros(256, 512, dtype=torch.float8_e4m3fn), "weight_scale": torch.zeros(256, 1, dtype=torch.bfloat16)},
             F8, "float-quantized")
    eng.classify_decompress(j)
    assert (j.kind, j.shape) == ("dq8c", (256, 512))
    j = _job({"weight_packed": torch.zeros(256, 256, dtype=torch.uint8), "weight_scale": torch.zeros(256, 32, dtype=torch.float8_e4m3fn),
              "weight_global_scale": torch.ones(1, dtype=torch.float32)}, F4, "nvfp4-pack-quantized")
    eng.classify_decompress(j)
    assert (j.kind, j.shape) == ("dq4f", (256, 512))
    j = _job({"weight_packed": torch.zeros(256, 256, dtype=torch.uint8), "weight_scale": torch.zeros(256, 32, dtype=torch.float8_e4m3fn),
              "weight_global_scale": torch.ones(1, dtype=torch.float32), "weight_zero_point": torch.zeros(256, 32, dtype=torch.float8_e4m3fn)},
             F4, "nvfp4-pack-quantized")
    eng.classify_decompress(j)
    assert j.kind == "generic", "a stored zero point takes the per-tensor dequantize"


def test_every_whole_shard_kind_can_be_planned():
    assert set(E._PLANNED_KINDS) == {"rotq4", "q4", "dq4", "q8c", "dq8c", "q4f", "dq4f"}
    assert all(dt in E._ITEMSIZE for dt in (torch.float8_e4m3fn, torch.uint8, torch.int32, torch.bfloat16))


def test_arena_views_are_aligned_and_disjoint():
    a = E._Arena(E._up(300 * 2) + E._up(7 * 64 * 4) + E._up(33))
    x = a.take((3, 100), torch.bfloat16)
    y = a.take((7, 64), torch.int32)
    z = a.take((33,), torch.uint8)
    assert x.is_contiguous() and y.is_contiguous() and z.is_contiguous()
    ptrs = [t.data_ptr() - a.buf.data_ptr() for t in (x, y, z)]
    assert ptrs == [0, E._up(600), E._up(600) + E._up(7 * 64 * 4)] and all(p % 256 == 0 for p in ptrs)
    x.fill_(1), y.fill_(2), z.fill_(3)
    assert float(x.sum()) == 300 and int(y.sum()) == 2 * 448 and int(z.sum()) == 99


def test_g_idx_column_order_is_remembered_per_tensor_state():
    F._G_IDX_UNSET.clear()
    g = torch.full((64,), -1, dtype=torch.int32)
    assert F._resolve_g_idx(g, 16, 64) is None
    assert len(F._G_IDX_UNSET) == 1
    assert F._resolve_g_idx(g, 16, 64) is None and len(F._G_IDX_UNSET) == 1, "same state: no second read-back"
    g.copy_(torch.arange(64, dtype=torch.int32) // 16)  # filled in place: a new version of the same storage
    assert F._resolve_g_idx(g, 16, 64) is g
    g[5] = -1
    assert F._resolve_g_idx(g, 16, 64) is None
