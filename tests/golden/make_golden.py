"""Generate the golden fixtures in this folder by running the reference implementation.

Usage (only where the reference checkout is available; the fixtures are committed so the
test-suite never needs it):

    python tests/golden/make_golden.py /path/to/compressed-tensors [fixture-name]

The reference is imported from ``<checkout>/src`` with a stub for its build-generated
``version`` module, in eager mode (``TORCHDYNAMO_DISABLE=1``).  Every fixture is a dict of
small tensors holding seeded inputs and the reference's outputs for them.
"""
import itertools
import os
import sys
import types

os.environ.setdefault("TORCHDYNAMO_DISABLE", "1")
os.environ.setdefault("HF_HUB_OFFLINE", "1")

if len(sys.argv) < 2:
    sys.exit(__doc__)
REF = sys.argv[1]
_v = types.ModuleType("compressed_tensors.version")
_v.__version__ = _v.version = "0.0.0"
_v.__all__ = ["__version__", "version"]
sys.modules["compressed_tensors.version"] = _v
sys.path.insert(0, os.path.join(REF, "src"))

import torch  # noqa: E402

import compressed_tensors  # noqa: E402

assert compressed_tensors.__file__.startswith(REF), compressed_tensors.__file__

from compressed_tensors.compressors.quantized_compressors.fp4_quantized import (  # noqa: E402
    NVFP4PackedCompressor,
    pack_fp4_to_uint8,
    unpack_fp4_from_uint8,
)
from compressed_tensors.compressors.quantized_compressors.naive_quantized import (  # noqa: E402
    NaiveQuantizationCompressor,
)
from compressed_tensors.compressors.quantized_compressors.pack_quantized import (  # noqa: E402
    PackedQuantizationCompressor,
    pack_to_int32,
    unpack_from_int32,
)
from compressed_tensors.compressors.sparse_compressors.sparse_24_bitmask import (  # noqa: E402
    get_24_bytemasks,
    sparse24_bitmask_compress,
    sparse24_bitmask_decompress,
)
from compressed_tensors.compressors.sparse_compressors.sparse_bitmask import (  # noqa: E402
    bitmask_compress,
    bitmask_decompress,
)
from compressed_tensors.quantization import QuantizationArgs  # noqa: E402
from compressed_tensors.quantization.lifecycle.forward import (  # noqa: E402
    dequantize,
    fake_quantize,
    quantize,
)
from compressed_tensors.quantization.utils.helpers import (  # noqa: E402
    calculate_qparams,
    compute_dynamic_scales_and_zp,
    generate_gparam,
)
from compressed_tensors.transform import TransformArgs, TransformScheme  # noqa: E402
from compressed_tensors.transform.factory.hadamard import HadamardFactory  # noqa: E402
from compressed_tensors.transform.factory.random_hadamard import RandomHadamardFactory  # noqa: E402
from compressed_tensors.transform.utils.hadamard import (  # noqa: E402
    deterministic_hadamard_matrix,
    random_hadamard_matrix,
)

OUT = os.path.dirname(os.path.abspath(__file__))


def weights(gen, rows, cols, dtype, std=0.02):
    """N(0, std) weights with a few rows of awkward values (zeros, signed zero, ties, extremes)."""
    w = (torch.randn(rows, cols, generator=gen) * std).to(dtype)
    w[0, : cols // 2] = 0.0
    w[1, ::3] = -0.0
    w[2] = torch.linspace(-1.0, 1.0, cols).to(dtype)  # many exact ties after scaling
    w[3, :8] = torch.tensor([3.0, -3.0, 1e-6, -1e-6, 0.5, -0.5, 100.0, -100.0]).to(dtype)
    w[4] = 0.0  # an all-zero row: scale clamps to eps / 0.125
    return w


def group_minmax(x, g):
    v = x.unflatten(-1, (x.shape[-1] // g, g))
    return torch.amin(v, dim=-1), torch.amax(v, dim=-1)


def gen_int():
    """int4/int8, symmetric/asymmetric, tensor/channel/group, bf16/fp16/fp32."""
    out = {}
    gen = torch.Generator().manual_seed(0)
    cases = [
        ("w4_sym_g128_bf16", 4, True, "group", 128, torch.bfloat16),
        ("w4_asym_g128_bf16", 4, False, "group", 128, torch.bfloat16),
        ("w4_sym_g32_bf16", 4, True, "group", 32, torch.bfloat16),
        ("w8_sym_g128_bf16", 8, True, "group", 128, torch.bfloat16),
        ("w8_sym_channel_bf16", 8, True, "channel", None, torch.bfloat16),
        ("w8_asym_channel_bf16", 8, False, "channel", None, torch.bfloat16),
        ("w4_sym_tensor_bf16", 4, True, "tensor", None, torch.bfloat16),
        ("w4_sym_g128_fp32", 4, True, "group", 128, torch.float32),
        ("w4_asym_g64_fp16", 4, False, "group", 64, torch.float16),
        ("w4_sym_channel_fp32", 4, True, "channel", None, torch.float32),
    ]
    for name, bits, sym, strategy, g, dtype in cases:
        x = weights(gen, 16, 256, dtype)
        args = QuantizationArgs(num_bits=bits, symmetric=sym, strategy=strategy, group_size=g)
        if strategy == "group":
            mn, mx = group_minmax(x, g)
        elif strategy == "channel":
            mn, mx = torch.amin(x, dim=-1, keepdim=True), torch.amax(x, dim=-1, keepdim=True)
        else:
            mn, mx = torch.aminmax(x)
        scale, zp = calculate_qparams(mn, mx, args)
        q8 = quantize(x, scale, zp, args, dtype=torch.int8)
        packed = pack_to_int32(q8, bits)
        d = {
            "x": x, "min": mn, "max": mx, "scale": scale, "zp": zp,
            "q_int8": q8,
            "q_float": quantize(x, scale, zp, args),
            "packed": packed,
            "unpacked": unpack_from_int32(packed, bits, x.shape),
            "dequant": dequantize(q8, scale, zp, args),
            "dequant_noargs": dequantize(q8, scale, zp) if strategy != "tensor" else dequantize(q8, scale, zp, args),
            "fake": fake_quantize(x, scale, zp, args),
            "bits": torch.tensor(bits), "sym": torch.tensor(sym), "group": torch.tensor(g or 0),
        }
        comp = PackedQuantizationCompressor()
        cd = comp.compress_weight(x, scale, args, zero_point=zp)
        for k, v in cd.items():
            d["c_" + k] = v
        cd["weight_scale"] = scale
        d["decompressed"] = comp.decompress_weight(cd, args)
        out[name] = d
    # activation ordering: groups assigned by a permuted column map
    x = weights(gen, 16, 256, torch.bfloat16)
    g = 64
    perm = torch.randperm(256, generator=gen)
    g_idx = torch.empty(256, dtype=torch.int32)
    g_idx[perm] = (torch.arange(256) // g).to(torch.int32)
    args = QuantizationArgs(num_bits=4, symmetric=True, strategy="group", group_size=g, actorder="group")
    xs = x.index_select(-1, torch.argsort(g_idx))
    mn, mx = group_minmax(xs, g)
    scale, zp = calculate_qparams(mn, mx, args)
    q8 = quantize(x, scale, zp, args, dtype=torch.int8, g_idx=g_idx)
    out["w4_sym_g64_actorder"] = {
        "x": x, "scale": scale, "zp": zp, "g_idx": g_idx, "q_int8": q8,
        "dequant": dequantize(q8, scale, zp, args, g_idx=g_idx),
        "fake": fake_quantize(x, scale, zp, args, g_idx=g_idx),
        "bits": torch.tensor(4), "sym": torch.tensor(True), "group": torch.tensor(g),
    }
    # exact words asserted by the reference's own pack test
    for bits, vals in ((4, [-8, -7, -6, -5, -4, -3, -2, -1]), (8, [1, 2, 3, 4]), (4, [1, 2, 3]), (2, list(range(-2, 2)) * 5)):
        v = torch.tensor([vals], dtype=torch.int8)
        out[f"pack_known_{bits}_{len(vals)}"] = {"value": v, "packed": pack_to_int32(v, bits), "bits": torch.tensor(bits)}
    # packing of zero points along dim 0
    zp = torch.randint(-8, 8, (20, 6), generator=gen, dtype=torch.int8)
    pz = pack_to_int32(zp, 4, packed_dim=0)
    out["pack_dim0"] = {"value": zp, "packed": pz.contiguous(), "unpacked": unpack_from_int32(pz, 4, zp.shape, packed_dim=0)}
    torch.save(out, os.path.join(OUT, "int_quant.pt"))


def gen_fp8():
    out = {}
    gen = torch.Generator().manual_seed(1)
    args_c = QuantizationArgs(num_bits=8, type="float", symmetric=True, strategy="channel")
    args_t = QuantizationArgs(num_bits=8, type="float", symmetric=True, strategy="tensor")
    args_tok = QuantizationArgs(num_bits=8, type="float", symmetric=True, strategy="token", dynamic=True)
    args_b = QuantizationArgs(num_bits=8, type="float", symmetric=True, strategy="block", block_structure=[16, 64])
    for dtype, sdt, tag in ((torch.bfloat16, None, "bf16"), (torch.bfloat16, torch.float32, "bf16_f32scale"),
                            (torch.float16, None, "fp16"), (torch.float32, None, "fp32")):
        x = weights(gen, 32, 256, dtype)
        xs = x if sdt is None else x.to(sdt)
        mn, mx = torch.amin(xs, dim=-1, keepdim=True), torch.amax(xs, dim=-1, keepdim=True)
        scale, zp = calculate_qparams(mn, mx, args_c)
        q = quantize(x, scale, zp, args_c, dtype=torch.float8_e4m3fn)
        out["channel_" + tag] = {
            "x": x, "scale": scale, "zp": zp, "q": q, "q_float": quantize(x, scale, zp, args_c),
            "dequant": dequantize(q, scale, zp, args_c), "dequant_noargs": dequantize(q, scale),
            "fake": fake_quantize(x, scale, zp, args_c),
        }
        c = NaiveQuantizationCompressor()
        cd = c.compress_weight(x, scale, args_c, zero_point=zp)
        out["channel_" + tag]["c_weight"] = cd["weight"]
        cd["weight_scale"] = scale
        out["channel_" + tag]["decompressed"] = c.decompress_weight(cd, args_c)
    x = weights(gen, 32, 256, torch.bfloat16)
    scale, zp = calculate_qparams(*torch.aminmax(x), args_t)
    q = quantize(x, scale, zp, args_t, dtype=torch.float8_e4m3fn)
    out["tensor_bf16"] = {"x": x, "scale": scale, "zp": zp, "q": q, "dequant": dequantize(q, scale, zp, args_t),
                          "fake": fake_quantize(x, scale, zp, args_t)}
    # dynamic per token, with outlier channels
    act = torch.randn(2, 24, 256, generator=gen)
    idx = torch.randperm(256, generator=gen)[:3]
    act[..., idx] *= 20
    act[0, 0] = 0.0
    act = act.to(torch.bfloat16)
    scale, zp = compute_dynamic_scales_and_zp(act, args_tok, module=None)
    q = quantize(act, scale, zp, args_tok, dtype=torch.float8_e4m3fn)
    out["token_bf16"] = {"x": act, "scale": scale, "zp": zp, "q": q, "dequant": dequantize(q, scale, zp, args_tok),
                         "fake": fake_quantize(act, scale, zp, args_tok)}
    # 2-D input under TOKEN collapses to one scale for the whole tensor
    s2, z2 = compute_dynamic_scales_and_zp(act[0], args_tok, module=None)
    out["token_2d"] = {"x": act[0], "scale": s2, "zp": z2}
    # block strategy
    x = weights(gen, 32, 256, torch.bfloat16)
    xb = x.reshape(2, 16, 4, 64).transpose(1, 2)
    mn, mx = torch.amin(xb, dim=(-1, -2)), torch.amax(xb, dim=(-1, -2))
    scale, zp = calculate_qparams(mn, mx, args_b)
    q = quantize(x, scale, zp, args_b, dtype=torch.float8_e4m3fn)
    out["block_bf16"] = {"x": x, "scale": scale, "zp": zp, "q": q, "dequant": dequantize(q, scale, zp, args_b),
                         "fake": fake_quantize(x, scale, zp, args_b)}
    # e4m3 rounding probe: every bf16 value in a range, unit scale
    allv = torch.arange(0x3000, 0x4400, dtype=torch.int32).to(torch.int16).view(torch.bfloat16).reshape(1, -1)
    allv = torch.cat([allv, -allv], dim=0)
    one = torch.ones(1, dtype=torch.bfloat16)
    out["e4m3_probe"] = {"x": allv, "scale": one, "q": quantize(allv, one, None, args_t, dtype=torch.float8_e4m3fn)}
    torch.save(out, os.path.join(OUT, "fp8_quant.pt"))


def gen_nvfp4():
    out = {}
    gen = torch.Generator().manual_seed(2)
    args = QuantizationArgs(num_bits=4, type="float", symmetric=True, strategy="tensor_group", group_size=16)
    for tag, rows, cols in (("a", 24, 256), ("b", 8, 64)):
        x = weights(gen, rows, cols, torch.bfloat16)
        x[3, :8] = x[3, :8] / 50  # keep the global scale dominated by the N(0, .02) body
        mn, mx = torch.aminmax(x)
        gs = generate_gparam(mn, mx)
        gmn, gmx = group_minmax(x, 16)
        scale, zp = calculate_qparams(gmn, gmx, args, global_scale=gs)
        q = quantize(x, scale, zp, args, global_scale=gs)
        packed = pack_fp4_to_uint8(q)
        unpacked = unpack_fp4_from_uint8(packed, rows, cols)
        comp = NVFP4PackedCompressor()
        cd = comp.compress_weight(x, scale, gs, args, zero_point=zp)
        out[tag] = {
            "x": x, "min": mn.reshape(1), "max": mx.reshape(1), "global_scale": gs, "gmin": gmn, "gmax": gmx,
            "scale": scale, "zp": zp, "q": q, "packed": packed, "unpacked": unpacked,
            "dequant": dequantize(unpacked, scale, global_scale=gs, dtype=torch.bfloat16),
            "fake": fake_quantize(x, scale, zp, args, global_scale=gs),
            "c_weight_packed": cd["weight_packed"],
            "decompressed": comp.decompress_weight({"weight_packed": packed, "weight_scale": scale,
                                                    "weight_global_scale": gs}, args),
        }
    # threshold probe for the e2m1 cast: a fine sweep of fp32 values through unit scales
    sweep = torch.cat([torch.linspace(-7, 7, 1121), torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, -0.25, -0.0, 0.0, -1e-3])])
    sweep = torch.nn.functional.pad(sweep, (0, 1136 - sweep.numel())).reshape(1, -1)
    one = torch.ones(1, 1136 // 16, dtype=torch.float8_e4m3fn)
    gs1 = torch.ones(1)
    q = quantize(sweep, one, None, args, global_scale=gs1)
    out["e2m1_probe"] = {"x": sweep, "scale": one, "global_scale": gs1, "q": q, "packed": pack_fp4_to_uint8(q)}
    torch.save(out, os.path.join(OUT, "nvfp4.pt"))


def gen_sparse():
    out = {}
    gen = torch.Generator().manual_seed(3)
    for dtype, tag in ((torch.bfloat16, "bf16"), (torch.float16, "fp16"), (torch.float32, "fp32"), (torch.float8_e4m3fn, "e4m3")):
        for cols in (64, 13):
            x = torch.randn(12, cols, generator=gen) * 0.5
            x[torch.rand(12, cols, generator=gen) < 0.5] = 0.0
            x[1, ::2] = -0.0
            x[5] = 0.0
            x = x.to(dtype)
            values, bitmask, row_offsets = bitmask_compress(x)
            out[f"bitmask_{tag}_{cols}"] = {
                "x": x, "values": values, "bitmask": bitmask, "row_offsets": row_offsets,
                "dense": bitmask_decompress(values, bitmask, list(x.shape)),
            }
    for dtype, tag in ((torch.bfloat16, "bf16"), (torch.float32, "fp32"), (torch.int8, "int8"), (torch.float8_e4m3fn, "e4m3")):
        if dtype == torch.int8:
            x = torch.randint(-128, 128, (16, 64), generator=gen, dtype=torch.int8)
        else:
            x = torch.randn(16, 64, generator=gen)
            x[0] = torch.round(x[0] * 2) / 2  # many ties
            x[1] = 0.0
            x[2, ::2] = 1.0
            x = x.to(dtype)
        mask = get_24_bytemasks(x)
        values, bitmask = sparse24_bitmask_compress(x)
        out[f"s24_{tag}"] = {"x": x, "mask": mask, "values": values, "bitmask": bitmask,
                             "dense": sparse24_bitmask_decompress(values, bitmask, list(x.shape))}
    # keep-mask for every weak ordering of four magnitudes (dense ranks 0..3)
    pats = [p for p in itertools.product(range(4), repeat=4) if set(p) == set(range(len(set(p))))]
    ranks = torch.tensor(pats, dtype=torch.float32)
    out["s24_rank_patterns"] = {"ranks": ranks.to(torch.int8), "mask": get_24_bytemasks(ranks),
                                "mask_int8": get_24_bytemasks(ranks.to(torch.int8)),
                                "mask_bf16": get_24_bytemasks(ranks.to(torch.bfloat16))}
    torch.save(out, os.path.join(OUT, "sparse.pt"))


def gen_hadamard():
    out = {}
    for n in (16, 64, 128, 256):
        out[f"det_{n}"] = {"H": deterministic_hadamard_matrix(n, torch.float64).to(torch.int8)}
        g = torch.Generator().manual_seed(42)
        out[f"rand_{n}_seed42"] = {"H": random_hadamard_matrix(n, torch.float64, gen=g).to(torch.int8)}
    gen = torch.Generator().manual_seed(4)
    for tag, fac_cls, seed in (("hadamard", HadamardFactory, None), ("random", RandomHadamardFactory, 7)):
        for location, inverse in (("weight_input", False), ("weight_input", True), ("weight_output", False), ("weight_output", True)):
            for dtype in (torch.bfloat16, torch.float32):
                o, i = (16, 256) if location == "weight_input" else (256, 16)
                lin = torch.nn.Linear(i, o, bias=False, dtype=dtype)
                lin.weight.data = weights(gen, o, i, dtype)
                scheme = TransformScheme(type=tag if tag == "hadamard" else "random-hadamard", head_dim=128,
                                         apply=[TransformArgs(targets=["Linear"], location=location, inverse=inverse)])
                fac = fac_cls("t", scheme, seed=seed)
                tr = fac.create_transform(lin, scheme.apply[0])
                w0 = lin.weight.data.clone()
                with torch.no_grad():
                    w1 = tr(lin.weight)
                name = f"{tag}_{location}_{'inv' if inverse else 'fwd'}_{str(dtype).split('.')[-1]}"
                out[name] = {"w": w0, "out": w1.detach(), "matrix": tr.weight.detach().to(torch.int8)}
    torch.save(out, os.path.join(OUT, "hadamard.pt"))


def gen_hadamard_online():
    """Activation-side (input / output) Hadamard transforms at the scheme's runtime precision (fp32)."""
    out = {}
    gen = torch.Generator().manual_seed(5)
    for tag, fac_cls, seed in (("hadamard", HadamardFactory, None), ("random", RandomHadamardFactory, 7)):
        for location in ("input", "output"):
            for inverse in (False, True):
                for dtype in (torch.bfloat16, torch.float32):
                    i, o = (256, 16) if location == "input" else (16, 256)
                    lin = torch.nn.Linear(i, o, bias=False, dtype=dtype)
                    scheme = TransformScheme(type=tag if tag == "hadamard" else "random-hadamard", head_dim=128,
                                             apply=[TransformArgs(targets=["Linear"], location=location, inverse=inverse)])
                    fac = fac_cls("t", scheme, seed=seed)
                    tr = fac.create_transform(lin, scheme.apply[0])
                    x = torch.randn(2, 3, 256, generator=gen).to(dtype)
                    with torch.no_grad():
                        y = tr(x)
                    name = f"{tag}_{location}_{'inv' if inverse else 'fwd'}_{str(dtype).split('.')[-1]}"
                    out[name] = {"x": x, "out": y.detach(), "matrix": tr.weight.detach().to(torch.int8)}
    torch.save(out, os.path.join(OUT, "hadamard_online.pt"))


def gen_marlin24():
    """Marlin24Compressor on 2:4-pruned weights: the quantized codes, the CUTLASS 2:4 compaction with its reordered
    meta, and the final packed tensors, for group-128 and channel scales at 4 and 8 bits."""
    from compressed_tensors.compressors.sparse_quantized_compressors.marlin_24 import Marlin24Compressor, compress_weight_24
    from compressed_tensors.quantization import QuantizationScheme
    from compressed_tensors.quantization.utils import calculate_qparams

    out = {}
    gen = torch.Generator().manual_seed(24)
    for bits in (4, 8):
        for strategy, rows, cols in (("group", 64, 256), ("channel", 128, 128), ("group", 64, 128), ("group", 64, 512)):
            w = weights(gen, rows, cols, torch.float32, std=0.05)
            w[:, 5] = 0.0  # incidental zeros: runs with three zeros
            w[3, :] = 0.0  # and runs that are all zero
            a = w.abs().reshape(-1, 4)
            keep = torch.zeros_like(a, dtype=torch.bool).scatter_(1, a.topk(2, dim=1).indices, True)
            w = (w.reshape(-1, 4) * keep).reshape(rows, cols)
            args = QuantizationArgs(num_bits=bits, symmetric=True, strategy=strategy, group_size=128 if strategy == "group" else None)
            if strategy == "group":
                mn, mx = group_minmax(w, 128)
            else:
                mn, mx = w.amin(dim=1, keepdim=True), w.amax(dim=1, keepdim=True)
            scale, zp = calculate_qparams(mn, mx, args)
            q = quantize(x=w.to(torch.float16), scale=scale.to(torch.float16), zero_point=None, args=args)
            sparse, meta = compress_weight_24(q)
            from compressed_tensors.utils.semi_structured_conversions import sparse_semi_structured_to_dense_cutlass
            dense_back = sparse_semi_structured_to_dense_cutlass(sparse, meta)
            scheme = QuantizationScheme(targets=["Linear"], weights=args)
            packed = Marlin24Compressor().compress({"l.weight": w.clone(), "l.weight_scale": scale.clone()}, {"l": scheme})
            out[f"w{bits}_{strategy}_{rows}x{cols}"] = {
                "weight": w.to(torch.float16), "scale": scale, "bits": torch.tensor(bits), "group": torch.tensor(128 if strategy == "group" else 0),
                "q": q.to(torch.int8), "sparse": sparse.to(torch.int8), "meta_reordered": meta, "dense_back": dense_back.to(torch.int8),
                "weight_packed": packed["l.weight_packed"], "scale_packed": packed["l.scale_packed"], "meta": packed["l.meta"]}
    from compressed_tensors.utils.permutations_24 import get_permutations_24
    for bits in (4, 8):
        perm, scale_perm, scale_perm_single = get_permutations_24(bits)
        out[f"permutations_{bits}"] = {"perm": perm.to(torch.int16), "scale_perm": torch.tensor(scale_perm, dtype=torch.int16),
                                       "scale_perm_single": torch.tensor(scale_perm_single, dtype=torch.int16)}
    torch.save(out, os.path.join(OUT, "marlin24.pt"))


def gen_hadamard_randomize():
    """randomize=True: the Hadamard matrix with its rows and columns permuted (factory/hadamard.py:62, :104-108)."""
    out = {}
    gen = torch.Generator().manual_seed(6)
    for tag, fac_cls in (("hadamard", HadamardFactory), ("random", RandomHadamardFactory)):
        for location in ("weight_input", "weight_output", "input"):
            for inverse in (False, True):
                i, o = (16, 256) if location == "weight_output" else (256, 16)
                lin = torch.nn.Linear(i, o, bias=False, dtype=torch.bfloat16)
                scheme = TransformScheme(type=tag if tag == "hadamard" else "random-hadamard", head_dim=128, randomize=True,
                                         apply=[TransformArgs(targets=["Linear"], location=location, inverse=inverse)])
                fac = fac_cls("t", scheme, seed=11)
                tr = fac.create_transform(lin, scheme.apply[0])
                x = weights(gen, o, i, torch.bfloat16) if location != "input" else torch.randn(3, 256, generator=gen).to(torch.bfloat16)
                with torch.no_grad():
                    y = tr(x)
                out[f"{tag}_{location}_{'inv' if inverse else 'fwd'}"] = {
                    "x": x, "out": y.detach(), "matrix": tr.weight.detach().to(torch.int8), "perm": tr.perm.detach().clone()}
    torch.save(out, os.path.join(OUT, "hadamard_randomize.pt"))


def gen_hadamard_embedding():
    """Transforms fused into an Embedding weight (matrix.py:121-126: the weight is applied as y = x W, so the sides
    swap relative to Linear)."""
    out = {}
    gen = torch.Generator().manual_seed(8)
    for tag, fac_cls, seed in (("random", RandomHadamardFactory, 7),):
        for location in ("weight_input", "weight_output"):
            for inverse in (False, True):
                emb = torch.nn.Embedding(128, 128, dtype=torch.bfloat16)
                emb.weight.data = weights(gen, 128, 128, torch.bfloat16)
                scheme = TransformScheme(type=tag if tag == "hadamard" else "random-hadamard", head_dim=128,
                                         apply=[TransformArgs(targets=["Embedding"], location=location, inverse=inverse)])
                tr = fac_cls("t", scheme, seed=seed).create_transform(emb, scheme.apply[0])
                w0 = emb.weight.data.clone()
                with torch.no_grad():
                    w1 = tr(emb.weight)
                out[f"{tag}_{location}_{'inv' if inverse else 'fwd'}"] = {"w": w0, "out": w1.detach()}
    torch.save(out, os.path.join(OUT, "hadamard_embedding.pt"))


def gen_mxfp4():
    """quantization/utils/mxfp4_utils.py on EVERY bf16 bit pattern and every uint8 exponent."""
    from compressed_tensors.quantization.utils.mxfp4_utils import (
        convert_mxfp4_exp_scale,
        generate_mxfp4_scales,
        round_to_power_2,
    )

    bits = torch.arange(65536, dtype=torch.int32).to(torch.uint16)
    x = bits.view(torch.bfloat16)
    exps = torch.arange(256, dtype=torch.int32).to(torch.uint8)
    out = {
        "all_bf16": {"round_pow2_bits": round_to_power_2(x).view(torch.uint16).to(torch.int32).to(torch.uint16),
                     "scales": generate_mxfp4_scales(x)},
        "all_exponents": {"bf16": convert_mxfp4_exp_scale(exps, torch.bfloat16),
                          "f16": convert_mxfp4_exp_scale(exps, torch.float16),
                          "f32": convert_mxfp4_exp_scale(exps, torch.float32)},
    }
    torch.save(out, os.path.join(OUT, "mxfp4.pt"))


def gen_hadamard_full():
    """Transforms as wide as the whole dimension (no head_dim): n = 1024 and 2048, both factories, both weight sides.
    Only the first column of each matrix is stored (the random signs; all ones for the deterministic matrix)."""
    out = {}
    gen = torch.Generator().manual_seed(14)
    for n in (1024, 2048):
        for tag, fac_cls, seed in (("hadamard", HadamardFactory, None), ("random", RandomHadamardFactory, 7)):
            for location, inverse in (("weight_input", False), ("weight_input", True), ("weight_output", False), ("weight_output", True)):
                o, i = (8, n) if location == "weight_input" else (n, 8)
                lin = torch.nn.Linear(i, o, bias=False, dtype=torch.bfloat16)
                lin.weight.data = weights(gen, o, i, torch.bfloat16)
                scheme = TransformScheme(type=tag if tag == "hadamard" else "random-hadamard",
                                         apply=[TransformArgs(targets=["Linear"], location=location, inverse=inverse)])
                fac = fac_cls("t", scheme, seed=seed)
                tr = fac.create_transform(lin, scheme.apply[0])
                w0 = lin.weight.data.clone()
                with torch.no_grad():
                    w1 = tr(lin.weight)
                out[f"{tag}_{location}_{'inv' if inverse else 'fwd'}_{n}"] = {"w": w0, "out": w1.detach(), "signs": tr.weight.detach()[:, 0].to(torch.int8)}
    torch.save(out, os.path.join(OUT, "hadamard_full.pt"))


def gen_forward_quantize():
    """forward_quantize and the wrapped quantized forward (lifecycle/forward.py:355-452) on a Linear(256, 128):
    static group weights, dynamic per-token int8 / fp8 activations, static per-tensor int8 input and output."""
    from compressed_tensors.quantization import QuantizationScheme, QuantizationStatus
    from compressed_tensors.quantization.lifecycle.forward import forward_quantize
    from compressed_tensors.quantization.lifecycle.initialize import initialize_module_for_quantization

    out = {}
    gen = torch.Generator().manual_seed(21)
    w = weights(gen, 128, 256, torch.bfloat16)
    x = torch.randn(2, 24, 256, generator=gen).to(torch.bfloat16)
    x[..., 7] *= 20
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
    for name, sides in cases.items():
        scheme = QuantizationScheme(targets=["Linear"], **sides)
        lin = torch.nn.Linear(256, 128, bias=False, dtype=torch.bfloat16)
        lin.weight.data = w.clone()
        initialize_module_for_quantization(lin, scheme)
        wa = scheme.weights
        g = wa.group_size if wa.strategy == "group" else 256
        mn, mx = group_minmax(w, g)
        s, z = calculate_qparams(mn, mx, wa)
        lin.weight_scale.data = s.reshape(lin.weight_scale.shape).to(lin.weight_scale.dtype)
        if hasattr(lin, "weight_zero_point"):
            lin.weight_zero_point.data = z.reshape(lin.weight_zero_point.shape).to(lin.weight_zero_point.dtype)
        d = {"w": w, "x": x, "weight_scale": lin.weight_scale.data.clone()}
        if hasattr(lin, "weight_zero_point"):
            d["weight_zero_point"] = lin.weight_zero_point.data.clone()
        for side in ("input", "output"):
            a = getattr(scheme, f"{side}_activations")
            if a is not None and not a.dynamic:
                amax = x.abs().max() if side == "input" else torch.tensor(40.0, dtype=torch.bfloat16)
                sc, zp = calculate_qparams(-amax.reshape(1), amax.reshape(1), a)
                getattr(lin, f"{side}_scale").data = sc.reshape(getattr(lin, f"{side}_scale").shape).to(torch.bfloat16)
                d[f"{side}_scale"] = getattr(lin, f"{side}_scale").data.clone()
        lin.quantization_status = QuantizationStatus.FROZEN
        with torch.no_grad():
            d["fq_weight"] = forward_quantize(lin, lin.weight.data, "weight", scheme.weights)
            if scheme.input_activations is not None:
                d["fq_input"] = forward_quantize(lin, x, "input", scheme.input_activations)
            d["y"] = lin(x)
            lin.quantization_enabled = False
            d["y_disabled"] = lin(x)
        out[name] = d
    torch.save(out, os.path.join(OUT, "forward_quantize.pt"))


def gen_fp4_pack_all():
    """pack_fp4_to_uint8 on EVERY bf16 and f16 bit pattern (off-grid magnitudes, ties, infinities, NaNs) and on a
    float32 sweep; unpack_fp4_from_uint8 on every byte, in the three dense dtypes."""
    bits = torch.arange(65536, dtype=torch.int32).to(torch.uint16).reshape(256, 256)
    gen = torch.Generator().manual_seed(11)
    f32 = torch.cat([torch.linspace(-7, 7, 4001), torch.randn(4191, generator=gen) * 3]).reshape(64, 128)
    every_byte = torch.arange(256, dtype=torch.int32).to(torch.uint8).reshape(16, 16)
    out = {
        "bf16_packed": pack_fp4_to_uint8(bits.view(torch.bfloat16)),
        "f16_packed": pack_fp4_to_uint8(bits.view(torch.float16)),
        "f32": f32, "f32_packed": pack_fp4_to_uint8(f32),
        "unpacked_bf16": unpack_fp4_from_uint8(every_byte, 16, 32, dtype=torch.bfloat16),
        "unpacked_f16": unpack_fp4_from_uint8(every_byte, 16, 32, dtype=torch.float16),
        "unpacked_f32": unpack_fp4_from_uint8(every_byte, 16, 32, dtype=torch.float32),
    }
    torch.save(out, os.path.join(OUT, "fp4_pack_all.pt"))


TOY = dict(layers=2, hidden=128, intermediate=256, kv=128, vocab=64)


def toy_llama(seed: int, dtype=torch.bfloat16):
    """A two-layer module tree with Llama's Linear names and ratios (q/o hidden x hidden, k/v kv x hidden, gate/up
    intermediate x hidden, down hidden x intermediate, lm_head), seeded N(0, 0.02) weights.  No forward is needed."""
    from torch import nn

    def lin(o, i):
        return nn.Linear(i, o, bias=False, dtype=dtype)

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
            self.input_layernorm = nn.LayerNorm(TOY["hidden"], dtype=dtype)

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
    gen = torch.Generator().manual_seed(seed)
    with torch.no_grad():
        for name, p in m.named_parameters():
            if name.endswith("layernorm.weight") or name.endswith("layernorm.bias"):
                continue
            p.copy_((torch.randn(p.shape, generator=gen) * 0.02).to(dtype))
    return m


def gen_gparam_all():
    """generate_gparam for every positive finite bf16 and fp16 maximum (min = 0) and a float32 sample: the expression
    `FP8 max * FP4 max / amax` has a Python scalar on the left, and what torch does with that is part of the result."""
    out = {}
    bf = torch.arange(0, 0x7F80, dtype=torch.int32).to(torch.int16).view(torch.bfloat16)
    fh = torch.arange(0, 0x7C00, dtype=torch.int32).to(torch.int16).view(torch.float16)
    gen = torch.Generator().manual_seed(77)
    f32 = torch.cat([torch.rand(2048, generator=gen) * 4 + 1e-4, torch.randn(2048, generator=gen).abs() * 0.02 + 1e-7])
    for tag, mx in (("bf16", bf), ("f16", fh), ("f32", f32)):
        res = torch.cat([generate_gparam(torch.zeros((), dtype=mx.dtype), m) for m in mx])
        out[tag] = {"max": mx, "global_scale": res}
    # a negative minimum that dominates
    out["neg"] = {"min": -bf[1000:1100], "global_scale": torch.cat([generate_gparam(-m, m / 2) for m in bf[1000:1100]])}
    torch.save(out, os.path.join(OUT, "gparam_all.pt"))


def gen_model_compressor():
    """ModelCompressor on the toy model, the way a calibrated checkpoint is made: apply_transform_config (random Hadamard,
    block 128, weight_input) -> apply_quantization_config (W4A16 group 128) -> min-max scales through calculate_qparams ->
    ModelCompressor.compress / compress_model / decompress_model.  Second case: FP8 per-channel weights (float-quantized)
    stacked with sparse-24-bitmask on 2:4-pruned weights."""
    import copy

    from compressed_tensors.compressors import ModelCompressor
    from compressed_tensors.config import Sparse24BitMaskConfig
    from compressed_tensors.quantization import QuantizationConfig, QuantizationScheme, apply_quantization_config
    from compressed_tensors.transform import TransformConfig, apply_transform_config
    from compressed_tensors.utils import update_parameter_data

    out = {}

    def slim(original, compressed, compressed_inplace, decompressed):
        """What the tests compare, without storing a tensor twice: the in-place result must equal the state-dict result
        wherever both have a key (checked here), so only its key table is kept; of the decompressed model, the weights."""
        for k, v in compressed_inplace.items():
            if k in compressed:
                assert v.dtype == compressed[k].dtype and torch.equal(v.view(torch.uint8), compressed[k].view(torch.uint8)), k
        return {"original": original, "compressed": dict(compressed),
                "inplace_keys": {k: (str(v.dtype), tuple(v.shape)) for k, v in compressed_inplace.items()},
                "decompressed_keys": {k: (str(v.dtype), tuple(v.shape)) for k, v in decompressed.items()},
                "decompressed": {k: v for k, v in decompressed.items() if k.endswith(".weight")}}

    def calibrate(model):
        for name, mod in model.named_modules():
            scheme = getattr(mod, "quantization_scheme", None)
            if scheme is None or scheme.weights is None:
                continue
            a, w = scheme.weights, mod.weight.data
            g = a.group_size if a.strategy in ("group", "tensor_group") else w.shape[1]
            mn, mx = group_minmax(w, g)
            gs = None
            if a.strategy == "tensor_group":  # NVFP4: the fp32 global scale first, the e4m3 group scales under it
                gs = generate_gparam(w.min().reshape(1), w.max().reshape(1))
                update_parameter_data(mod, gs.reshape(mod.weight_global_scale.shape).to(mod.weight_global_scale.dtype), "weight_global_scale")
            s, z = calculate_qparams(mn, mx, a, global_scale=gs)
            update_parameter_data(mod, s.reshape(mod.weight_scale.shape).to(mod.weight_scale.dtype), "weight_scale")
            if hasattr(mod, "weight_zero_point"):
                update_parameter_data(mod, z.reshape(mod.weight_zero_point.shape).to(mod.weight_zero_point.dtype), "weight_zero_point")

    # ---- case 1: rotation + W4A16 pack-quantized
    model = toy_llama(31)
    original = {k: v.clone() for k, v in model.state_dict().items()}
    tcfg = TransformConfig(config_groups={"u": TransformScheme(type="random-hadamard", head_dim=128, apply=[
        TransformArgs(targets=["Linear"], ignore=["lm_head"], location="weight_input")])})
    apply_transform_config(model, tcfg)
    rotated = {k: v.clone() for k, v in model.state_dict().items()}
    qcfg = QuantizationConfig(config_groups={"group_0": QuantizationScheme(
        targets=["Linear"], weights=QuantizationArgs(num_bits=4, symmetric=True, strategy="group", group_size=128))},
        ignore=["lm_head"], format="pack-quantized")
    apply_quantization_config(model, qcfg)
    calibrate(model)
    calibrated = {k: v.clone() for k, v in model.state_dict().items()}
    mc = ModelCompressor(quantization_config=copy.deepcopy(qcfg))
    compressed = mc.compress(model)
    inplace = copy.deepcopy(model)
    mc2 = ModelCompressor(quantization_config=copy.deepcopy(qcfg))
    mc2.compress_model(inplace)
    compressed_inplace = {k: v.clone() for k, v in inplace.state_dict().items()}
    mc2.decompress_model(inplace)
    decompressed = {k: v.clone() for k, v in inplace.state_dict().items()}
    out["w4a16_rot"] = slim(original, compressed, compressed_inplace, decompressed)
    out["w4a16_rot"]["rotated_q_proj"] = rotated["model.layers.0.self_attn.q_proj.weight"]

    # ---- case 2: FP8 per-channel (float-quantized) stacked with 2:4 bitmask sparsity
    model = toy_llama(32)
    with torch.no_grad():
        for name, mod in model.named_modules():
            if isinstance(mod, torch.nn.Linear):
                w = mod.weight.data
                mask = get_24_bytemasks(w)
                mod.weight.data = torch.where(mask, w, torch.zeros((), dtype=w.dtype))
    original = {k: v.clone() for k, v in model.state_dict().items()}
    qcfg = QuantizationConfig(config_groups={"group_0": QuantizationScheme(
        targets=["Linear"], weights=QuantizationArgs(num_bits=8, type="float", symmetric=True, strategy="channel"))},
        ignore=["lm_head"], format="float-quantized")
    scfg = Sparse24BitMaskConfig(targets=["Linear"], ignore=["lm_head"], sparsity_structure="2:4")
    apply_quantization_config(model, qcfg)
    calibrate(model)
    calibrated = {k: v.clone() for k, v in model.state_dict().items()}
    mc = ModelCompressor(sparsity_config=scfg, quantization_config=copy.deepcopy(qcfg))
    compressed = mc.compress(model)
    inplace = copy.deepcopy(model)
    mc2 = ModelCompressor(sparsity_config=scfg, quantization_config=copy.deepcopy(qcfg))
    mc2.compress_model(inplace)
    compressed_inplace = {k: v.clone() for k, v in inplace.state_dict().items()}
    mc2.decompress_model(inplace)
    decompressed = {k: v.clone() for k, v in inplace.state_dict().items()}
    out["fp8_sparse24"] = slim(original, compressed, compressed_inplace, decompressed)

    # ---- case 3: the same weights and scales, FP8 per-channel alone (no sparsity config); `original` is case 2's
    model = toy_llama(32)
    model.load_state_dict(original)
    apply_quantization_config(model, qcfg)
    calibrate(model)
    mc = ModelCompressor(quantization_config=copy.deepcopy(qcfg))
    compressed = mc.compress(model)
    inplace = copy.deepcopy(model)
    mc2 = ModelCompressor(quantization_config=copy.deepcopy(qcfg))
    mc2.compress_model(inplace)
    compressed_inplace = {k: v.clone() for k, v in inplace.state_dict().items()}
    mc2.decompress_model(inplace)
    decompressed = {k: v.clone() for k, v in inplace.state_dict().items()}
    out["fp8_channel"] = slim({}, compressed, compressed_inplace, decompressed)
    # everything that is not a quantized weight (norms, embeddings, lm_head, scales) already sits in case 2
    out["fp8_channel"]["compressed"] = {k: v for k, v in compressed.items() if v.dtype == torch.float8_e4m3fn}
    out["fp8_channel"]["compressed_keys"] = {k: (str(v.dtype), tuple(v.shape)) for k, v in compressed.items()}

    # ---- case 4: the same weights as NVFP4 (nvfp4-pack-quantized); `original` is case 2's
    model = toy_llama(32)
    model.load_state_dict(original)
    qcfg4 = QuantizationConfig(config_groups={"group_0": QuantizationScheme(
        targets=["Linear"], weights=QuantizationArgs(num_bits=4, type="float", symmetric=True, strategy="tensor_group", group_size=16))},
        ignore=["lm_head"], format="nvfp4-pack-quantized")
    apply_quantization_config(model, qcfg4)
    calibrate(model)
    mc = ModelCompressor(quantization_config=copy.deepcopy(qcfg4))
    compressed = mc.compress(model)
    inplace = copy.deepcopy(model)
    mc2 = ModelCompressor(quantization_config=copy.deepcopy(qcfg4))
    mc2.compress_model(inplace)
    compressed_inplace = {k: v.clone() for k, v in inplace.state_dict().items()}
    mc2.decompress_model(inplace)
    decompressed = {k: v.clone() for k, v in inplace.state_dict().items()}
    out["nvfp4"] = slim({}, compressed, compressed_inplace, decompressed)
    out["nvfp4"]["compressed"] = {k: v for k, v in compressed.items()
                                  if k.endswith(("weight_packed", "weight_scale", "weight_global_scale"))}
    out["nvfp4"]["compressed_keys"] = {k: (str(v.dtype), tuple(v.shape)) for k, v in compressed.items()}
    torch.save(out, os.path.join(OUT, "model_compressor.pt"))


if __name__ == "__main__":
    only = sys.argv[2] if len(sys.argv) > 2 else None  # e.g. "mxfp4": regenerate one fixture
    for name, fn in (("int_quant", gen_int), ("fp8_quant", gen_fp8), ("nvfp4", gen_nvfp4), ("sparse", gen_sparse),
                     ("hadamard", gen_hadamard), ("hadamard_online", gen_hadamard_online), ("hadamard_randomize", gen_hadamard_randomize), ("hadamard_embedding", gen_hadamard_embedding), ("mxfp4", gen_mxfp4), ("marlin24", gen_marlin24),
                     ("fp4_pack_all", gen_fp4_pack_all), ("hadamard_full", gen_hadamard_full), ("forward_quantize", gen_forward_quantize), ("gparam_all", gen_gparam_all), ("model_compressor", gen_model_compressor)):
        if only is None or only == name:
            fn()
    for f in sorted(os.listdir(OUT)):
        if f.endswith(".pt"):
            print(f, os.path.getsize(os.path.join(OUT, f)))
