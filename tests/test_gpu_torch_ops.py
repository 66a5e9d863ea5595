"""The codec kernels as torch operators (torch.ops.ctb200.*): schema, fake implementations and dispatch checked by
torch.library.opcheck on real inputs; meta tensors go through the host mirror without touching the GPU."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _inputs():
    from compressed_tensors_b200 import ops

    g = torch.Generator(device="cuda").manual_seed(0)
    x = (torch.randn(64, 256, generator=g, device="cuda") * 0.02).to(torch.bfloat16)
    mn, mx = ops.minmax(x, 1, 128)
    s, z = ops.calculate_qparams(mn, mx, qtype=ops.QINT, bits=4, symmetric=False)
    words = ops.quantize(x, s, z, qtype=ops.QINT, bits=4, col_group=128, scale_row_stride=2, codec="pack32")
    codes = ops.quantize(x, s, z, qtype=ops.QINT, bits=4, col_group=128, scale_row_stride=2, out_dtype=torch.int8)
    signs = (torch.randint(0, 2, (128,), generator=g, device="cuda") * 2 - 1).to(torch.int8)
    sparse = x.clone()
    sparse[torch.rand(64, 256, generator=g, device="cuda") < 0.5] = 0
    v24, b24 = ops.sparse24_compress(x)
    vals, bm, _ = ops.bitmask_compress(sparse)
    fp4 = ops.unpack_fp4(torch.randint(0, 256, (64, 128), device="cuda", dtype=torch.uint8, generator=g), 64, 256)
    return {
        "quantize": (x, s, z, 0, 4, 128, 1, 2, None, "pack32", None, None),
        "dequantize": (words, s, z, 0, 4, 128, 1, 2, torch.bfloat16, "pack32", 256, None, None),
        "fake_quantize": (x, s, z, 0, 4, 128, 1, 2, torch.bfloat16, None, None),
        "absmax_quantize": (x, 0, 4, 128, "pack32", None, None, 128, signs, "float64"),
        "minmax": (x, 1, 128),
        "calculate_qparams": (mn, mx, 0, 4, True, None),
        "generate_gparam": (mn.min().reshape(1), mx.max().reshape(1)),
        "pack_int32": (codes, 4, 1),
        "unpack_int32": (words, 4, [64, 256], 1),
        "pack_fp4": (fp4,),
        "unpack_fp4": (ops.pack_fp4(fp4), 64, 256, torch.bfloat16),
        "pack_bitmasks": (sparse != 0,),
        "unpack_bitmasks": (bm, [64, 256]),
        "sparse24_mask": (x,),
        "sparse24_compress": (x,),
        "quantize_fp8_sparse24": (x, (x.abs().amax(dim=1) / 448).to(torch.bfloat16), None),
        "sparse24_decompress": (v24, b24, [64, 256]),
        "sparse24_decompress_dequantize_fp8": (*ops.quantize_fp8_sparse24(x, (x.abs().amax(dim=1) / 448).to(torch.bfloat16)),
                                               (x.abs().amax(dim=1) / 448).to(torch.bfloat16), [64, 256]),
        "bitmask_compress": (sparse,),
        "bitmask_decompress": (vals, bm, [64, 256]),
        "hadamard": (x, 128, signs, False, 0, "float64", True),
    }


def test_every_operator_is_registered_and_passes_opcheck():
    from compressed_tensors_b200 import torch_ops

    inputs = _inputs()
    assert set(inputs) == set(torch_ops.OPERATORS)
    for name in torch_ops.OPERATORS:
        op = getattr(torch.ops.ctb200, name).default
        tests = ("test_schema", "test_faketensor") if name == "bitmask_compress" else ("test_schema", "test_autograd_registration", "test_faketensor")
        if any(isinstance(a, torch.Tensor) and a.dtype == torch.float8_e4m3fn for a in inputs[name]):
            tests = tuple(t for t in tests if t != "test_schema")  # the schema check clones and compares inputs with ops float8 tensors lack
        torch.library.opcheck(op, inputs[name], test_utils=tests)


def test_operators_equal_the_direct_calls():
    from compressed_tensors_b200 import ops, torch_ops

    x = _inputs()["quantize"][0]
    mn, mx = torch_ops.minmax(x, 1, 128)
    s, z = torch_ops.calculate_qparams(mn, mx, qtype=ops.QINT, bits=4, symmetric=True)
    kw = dict(qtype=ops.QINT, bits=4, col_group=128, scale_row_stride=2, codec="pack32")
    assert torch.equal(torch_ops.quantize(x, s, None, **kw), ops.quantize(x, s, None, **kw))
    assert torch.equal(torch.ops.ctb200.hadamard(x, 128, None, False, 0, "float32", True), ops.hadamard(x, 128, precision=torch.float32))


def test_meta_tensors_go_through_the_host_mirror():
    """Shapes and dtypes of the reference-facing functions on meta tensors: nothing is launched."""
    from compressed_tensors_b200 import _lib as L
    from compressed_tensors_b200.compressors.quantized_compressors.pack_quantized import pack_to_int32
    from compressed_tensors_b200.compressors.sparse_compressors.sparse_24_bitmask import sparse24_bitmask_compress
    from compressed_tensors_b200.quantization import QuantizationArgs, fake_quantize, quantize

    n0 = L.launch_count()
    x = torch.empty(32, 256, dtype=torch.bfloat16, device="meta")
    s = torch.empty(32, 2, dtype=torch.bfloat16, device="meta")
    z = torch.empty(32, 2, dtype=torch.int8, device="meta")
    args = QuantizationArgs(num_bits=4, strategy="group", group_size=128)
    q = quantize(x, s, z, args, dtype=torch.int8)
    assert q.is_meta and q.dtype == torch.int8 and tuple(q.shape) == (32, 256)
    assert tuple(pack_to_int32(q, 4).shape) == (32, 32)
    assert fake_quantize(x, s, z, args).dtype == torch.bfloat16
    v, b = sparse24_bitmask_compress(x)
    assert v.is_meta and tuple(v.shape) == (32, 128) and tuple(b.shape) == (32, 32)
    assert L.launch_count() == n0
