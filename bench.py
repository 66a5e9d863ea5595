#!/usr/bin/env python
"""Benchmark of the tensor-codec hot path on B200.

Workload (BASELINE.json configs[4]): every Linear weight of a Llama-3-8B-shaped model (32 layers,
bf16, N(0, 0.02), synthetic), random-Hadamard rotation (block 128) fused with W4A16 int4 group-128
quantize + pack_to_int32, then unpack + dequantize.  Layers are dealt to the ranks in contiguous
blocks (strong scaling: the model is fixed, ranks split it); no collective is on the data path.

One "step" = ModelCompressor.compress_model (rotate + calibrate + quantize + pack, fused) then
ModelCompressor.decompress_model (unpack + dequantize) of the rank's share of a Llama-3-8B-shaped module tree.
value = bf16 bytes through both directions (2 x weight bytes, all ranks) / max-over-ranks device time.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import torch  # noqa: E402

METRIC = "bf16 weight GB/s through quantize+pack / unpack+dequant"
UNIT = "GB/s"
WORKLOAD = "llama3-8b-linears hadamard128+w4a16-g128 compress+decompress"
SEED = 0
ALG_BYTES_PER_ELEM = 2 + 0.5 + 2 / 128  # bf16 in, 4 bits out, one bf16 scale per 128 (either direction)
# dram__bytes_read.sum + dram__bytes_write.sum of rotquant128_tc_kernel per element, from the ncu capture of the two-layer
# case (872.45 MB + 204.32 MB over 436,207,616 elements; traffic grows in proportion to the elements processed)
NCU_TRAFFIC_BYTES_PER_ELEM = (872.452096e6 + 204.323584e6) / 436207616


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        return float(json.load(open(p))["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.proc = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={index}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            pass

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        out, _ = self.proc.communicate(timeout=10)
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0])); mx.append(float(f[1]))
            except ValueError:
                continue
            for n, v in zip(names, f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        # "under load": the upper half of the samples (idle samples before/after the region sit low)
        hi = sorted(sm)[len(sm) // 2:]
        return {"sm_mhz": statistics.median(hi), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


def make_weights(layers, device, shapes):
    ws = []
    for layer in layers:
        for j, (_, o, i) in enumerate(shapes):
            g = torch.Generator(device=device).manual_seed(SEED * 1000003 + layer * 16 + j)
            ws.append((torch.randn(o, i, generator=g, device=device, dtype=torch.float32) * 0.02).to(torch.bfloat16))
    return ws


def make_signs():
    g = torch.Generator().manual_seed(SEED)
    return (torch.randint(0, 2, (128,), generator=g) * 2 - 1).to(torch.int8)


def time_region(fn, steps, stream):
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record(stream)
    for _ in range(steps):
        fn()
    end.record(stream)
    end.synchronize()
    return start.elapsed_time(end) / 1e3  # seconds


def build_model(layers, shapes, weights):
    """A module tree with Llama's names: model.layers.<i>.self_attn.q_proj ... mlp.down_proj, one Linear per weight
    (no bias), the given tensors as parameters.  No forward pass is needed: the codec walks parameters."""
    nn = torch.nn
    root = nn.Module()
    root.add_module("model", nn.Module())
    root.model.add_module("layers", nn.ModuleList())
    it = iter(weights)
    for _ in layers:
        layer = nn.Module()
        for name, o, i in shapes:
            parent = layer
            *path, leaf = name.split(".")
            for p in path:
                if not hasattr(parent, p):
                    parent.add_module(p, nn.Module())
                parent = getattr(parent, p)
            lin = nn.Linear(i, o, bias=False, dtype=torch.bfloat16, device="meta")
            lin.weight = nn.Parameter(next(it), requires_grad=False)
            parent.add_module(leaf, lin)
        root.model.layers.append(layer)
    return root


def scheme_shard_leg(scheme, ctb, ModelCompressor, weights, layers, shapes, dev, peak, use_layers=8):
    """The same module tree (its first `use_layers` decoder layers) as a calibrated model of another scheme:
    "fp8" = FP8 per-channel float-quantized (3 algorithmic bytes per element each way), "nvfp4" = NVFP4
    nvfp4-pack-quantized (2.5625).  ModelCompressor.compress_model / decompress_model are each ONE launch over the whole
    shard (ctb_quantize_fp8_channel_batch / ctb_quantize_fp4_g16_batch and their inverses)."""
    q = ctb.quantization
    n = min(use_layers, len(layers))
    per = len(shapes)
    model = build_model(layers[:n], shapes, [w.clone() for w in weights[:n * per]])
    if scheme == "fp8":
        wargs, fmt, alg = q.QuantizationArgs(num_bits=8, type="float", symmetric=True, strategy="channel"), "float-quantized", 3.0
    else:
        wargs = q.QuantizationArgs(num_bits=4, type="float", symmetric=True, strategy="tensor_group", group_size=16)
        fmt, alg = "nvfp4-pack-quantized", 2.5625
    qcfg = q.QuantizationConfig(config_groups={"group_0": q.QuantizationScheme(targets=["Linear"], weights=wargs)},
                                ignore=["lm_head"], format=fmt)
    q.apply_quantization_config(model, qcfg)
    for m in model.modules():
        if getattr(m, "quantization_scheme", None) is not None and hasattr(m, "weight"):
            q.calibrate_weight_qparams(m)
    elems = sum(w.numel() for w in weights[:n * per])
    mc = ModelCompressor(quantization_config=qcfg)
    for _ in range(2):
        mc.compress_model(model)
        mc.decompress_model(model)
    torch.cuda.synchronize()
    mc.engine.record_kernel_times = True
    mc.engine.kernel_times.clear()
    launches0, reps = mc.engine.launches, 3
    t0 = time.perf_counter()
    for _ in range(reps):
        mc.compress_model(model)
        mc.decompress_model(model)
    torch.cuda.synchronize()
    wall = (time.perf_counter() - t0) / reps
    tc = sum(a.elapsed_time(b) for kind, a, b in mc.engine.kernel_times if kind == "compress") / 1e3 / reps
    td = sum(a.elapsed_time(b) for kind, a, b in mc.engine.kernel_times if kind == "decompress") / 1e3 / reps
    return {"layers": n, "elements": elems, "launches_per_cycle": (mc.engine.launches - launches0) / reps,
            "compress_ms": round(tc * 1e3, 3), "compress_frac": round(alg * elems / tc / 1e9 / peak, 3),
            "decompress_ms": round(td * 1e3, 3), "decompress_frac": round(alg * elems / td / 1e9 / peak, 3),
            "cycle_wall_ms": round(wall * 1e3, 2),
            "note": "kernel times from CUDA events around each launch; cycle_wall_ms includes the per-module host walk of the general path"}


def configs(pkg):
    """(transform config, quantization config) of the workload, built from `pkg` (this package or the reference)."""
    q, t = pkg.quantization, pkg.transform
    tcfg = t.TransformConfig(config_groups={"u": t.TransformScheme(type="random-hadamard", head_dim=128, apply=[
        t.TransformArgs(targets=["Linear"], ignore=["lm_head"], location="weight_input")])})
    qcfg = q.QuantizationConfig(config_groups={"group_0": q.QuantizationScheme(
        targets=["Linear"], weights=q.QuantizationArgs(num_bits=4, symmetric=True, strategy="group", group_size=128))},
        ignore=["lm_head"], format="pack-quantized")
    return tcfg, qcfg


def cpu_pass(ws, signs):
    """One pass of the path on the host through the oracle port (rotate, calibrate, quantize, pack, unpack, dequantize)."""
    from oracle import ref as orc
    out = 0
    for w in ws:
        rot = orc.hadamard(w, 128, signs=signs)
        mn, mx = orc.minmax(rot, 1, 128)
        scale, zp = orc.calculate_qparams(mn, mx, qtype=orc.QINT, bits=4, symmetric=True)
        kw = dict(qtype=orc.QINT, bits=4, col_group=128, row_group=1, scale_row_stride=w.shape[1] // 128)
        words = orc.pack_int32(orc.quantize(rot, scale, zp, out_dtype=torch.int8, **kw), 4)
        deq = orc.dequantize(orc.unpack_int32(words, 4, w.shape), scale, None, out_dtype=torch.bfloat16, **kw)
        out += deq.numel()
    return out


SAMPLE = (("self_attn.q_proj", 4096, 4096), ("self_attn.k_proj", 1024, 4096), ("mlp.gate_proj", 14336, 4096))
SAMPLE_TEXT = "q_proj 4096x4096 + k_proj 1024x4096 + gate_proj 14336x4096 of one decoder layer per step"


def cpu_sample():
    """Bounded sample of the workload for the CPU arm: q_proj, k_proj and gate_proj of one layer."""
    g = torch.Generator().manual_seed(SEED)
    return [(torch.randn(o, i, generator=g) * 0.02).to(torch.bfloat16) for _, o, i in SAMPLE]


class CpuArm:
    """The CPU side of the comparison on the bounded sample.  kind "reference": the reference package itself
    (oracle/_ref, installed from the checkout by __graft_entry__.build()) through its own public calls --
    apply_transform_config, min-max scales by calculate_qparams, ModelCompressor.compress_model and
    decompress_model -- in eager mode on all host threads.  kind "port": the C + OpenMP restatement, used only
    where the reference package is not present."""

    def __init__(self):
        from oracle import reference
        self.cores = os.cpu_count() or 1
        self.ws = cpu_sample()
        self.elems = sum(w.numel() for w in self.ws)
        self.kind = "reference" if reference.available() else "port"
        if self.kind == "reference":
            torch.set_num_threads(self.cores)
            self.ct = reference.load()
            import compressed_tensors.compressors, compressed_tensors.quantization, compressed_tensors.transform  # noqa: F401
        else:
            from oracle import ref as orc
            orc.build()
            orc.set_threads(self.cores)
            self.signs = make_signs()

    def one_pass(self):
        if self.kind == "port":
            return cpu_pass(self.ws, self.signs)
        import copy

        ct = self.ct
        from compressed_tensors.quantization.utils.helpers import calculate_qparams
        tcfg, qcfg = configs(ct)
        model = build_model([0], SAMPLE, [w.clone() for w in self.ws])
        with torch.no_grad():
            ct.transform.apply_transform_config(model, tcfg)
            ct.quantization.apply_quantization_config(model, qcfg)
            for m in model.modules():
                a = getattr(getattr(m, "quantization_scheme", None), "weights", None)
                if a is None:
                    continue
                grouped = m.weight.data.unflatten(-1, (-1, a.group_size))
                scale, _ = calculate_qparams(grouped.amin(-1), grouped.amax(-1), a)
                m.weight_scale.data = scale.reshape(m.weight_scale.shape).to(m.weight_scale.dtype)
            mc = ct.compressors.ModelCompressor(quantization_config=copy.deepcopy(qcfg))
            mc.compress_model(model)
            mc.decompress_model(model)
        return self.elems

    def time(self, steps, warmup):
        for _ in range(warmup):
            self.one_pass()
        t0 = time.perf_counter()
        for _ in range(steps):
            self.one_pass()
        dt = (time.perf_counter() - t0) / steps
        return dt, 2 * 2 * self.elems / dt / 1e9


def workload_config(layers, world, precision):
    return {"workload": WORKLOAD, "layers": layers, "partition": f"layers/{world}",
            "hadamard_accumulate": {"f64": "float64 butterfly (bit-identical to the reference)", "f32": "float32 butterfly",
                                    "tc": "tcgen05 bf16 x bf16 -> fp32 in TMEM"}[precision],
            "l2": "inputs larger than L2 (no flush needed)"}


_RESULT_FD = None


def quiet_stdout():
    """Libraries write to file descriptor 1 on their own (NCCL prints its version there at the first
    collective; progress bars of the reference).  The contract of this script is ONE JSON line on stdout, so
    descriptor 1 is pointed at stderr for the run and the result line goes to the saved descriptor."""
    global _RESULT_FD
    sys.stdout.flush()
    _RESULT_FD = os.dup(1)
    os.dup2(2, 1)


def emit(obj):
    line = (json.dumps(obj) + "\n").encode()
    if _RESULT_FD is None:
        sys.stdout.write(line.decode())
        sys.stdout.flush()
    else:
        sys.stdout.flush()
        os.write(_RESULT_FD, line)


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    arm = CpuArm()
    dt, val = arm.time(args.steps, args.warmup)
    cfg = workload_config(args.layers, args.gpus, args.precision)
    cfg["sample"] = SAMPLE_TEXT
    cfg["path"] = ("reference package: apply_transform_config -> calculate_qparams -> ModelCompressor.compress_model -> decompress_model"
                   if arm.kind == "reference" else "C + OpenMP restatement of the same calls")
    emit(({
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic", "config": cfg,
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": arm.cores, "kind": arm.kind, "sample": SAMPLE_TEXT},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def op_timer(out, peak):
    """Returns run(name, make_args, fn, dense_bytes, alg_bytes, per_set_bytes): times fn over a rotating set of
    distinct argument sets whose total exceeds 2x the L2 size, each call writing to output buffers of its own (every
    launch streams from and to HBM), replayed from a CUDA graph, with CUDA events on the current stream, and records
    us / dense GB/s / fraction of `peak` under out[name]."""
    l2 = 2 * 126 * 1024 * 1024

    def run(name, make_args, fn, dense_bytes, alg_bytes, per_set_bytes):
        nsets = int(max(2, min(16, -(-l2 // int(per_set_bytes)))))
        sets = [make_args() for _ in range(nsets)]
        for a in sets[:2]:
            fn(*a)
        torch.cuda.synchronize()
        reps = 3

        def sweep():
            # the results of a sweep stay alive until its end, so every call writes to memory of its own: an output
            # buffer handed back to the allocator and reused by the next call would be rewritten while still in L2
            held = [fn(*a) for a in sets]
            del held

        mode = "cuda graph"
        try:  # replay from a CUDA graph so that the host-side call overhead of these 5-50 us kernels is not what is timed
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                sweep()
            replay = graph.replay
        except Exception:  # ops that read a count back to the host cannot be captured
            torch.cuda.synchronize()
            replay, mode = sweep, "eager (host sync inside)"
        replay()
        torch.cuda.synchronize()
        st, en = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        st.record()
        for _ in range(reps):
            replay()
        en.record()
        en.synchronize()
        sec = st.elapsed_time(en) / 1e3 / (reps * nsets)
        out[name] = {"us": round(sec * 1e6, 2), "dense_gbs": round(dense_bytes / sec / 1e9, 1), "frac": round(alg_bytes / sec / 1e9 / peak, 3), "timed": mode}

    return run


def per_config_table(dev, peak):
    """Device-timed throughput of the other BASELINE.json configs (C1-C4) on their named shapes.  Each op runs
    over a rotating set of distinct input/output buffers whose total exceeds 2x the L2 size, so every launch
    streams from HBM.  GB/s is bf16 (dense-side) input bytes / time; frac = algorithmic bytes / time / peak."""
    from compressed_tensors_b200 import ops

    out = {}
    g = torch.Generator(device=dev).manual_seed(SEED + 1)

    def rnd(r, c, std=0.02):
        return (torch.randn(r, c, generator=g, device=dev) * std).to(torch.bfloat16)

    run = op_timer(out, peak)

    kw4 = dict(qtype=ops.QINT, bits=4, col_group=128)
    n = 4096 * 4096
    # what a single launch can reach on this much data: a plain device copy (torch's kernel) moving the same number of
    # bytes as the C1 / C2-weight kernels do (2.5 and 3 bytes per element of a 4096 x 4096 tensor, half read, half written)
    for tag, nbytes in (("copy_42MB_single_launch_ceiling", int(2.515625 * n)), ("copy_50MB_single_launch_ceiling", 3 * n)):
        run(tag, lambda nb=nbytes: (torch.empty(nb // 2, dtype=torch.uint8, device=dev).random_(0, 255),),
            lambda src: torch.empty_like(src).copy_(src), nbytes, nbytes, nbytes)
    run("c1_w4a16_calibrate_quantize_pack", lambda: (rnd(4096, 4096),),
        lambda w: ops.absmax_quantize(w, codec="pack32", **kw4), 2 * n, 2.515625 * n, 2.6 * n)
    def c1_dq_args():
        w = rnd(4096, 4096)
        return ops.absmax_quantize(w, codec="pack32", **kw4)
    run("c1_w4a16_unpack_dequantize", c1_dq_args,
        lambda p, sc: ops.dequantize(p, sc, None, scale_row_stride=32, out_dtype=torch.bfloat16, codec="pack32", cols=4096, **kw4),
        2 * n, 2.515625 * n, 2.6 * n)
    kw8 = dict(qtype=ops.QFLOAT, bits=8, col_group=4096)
    run("c2_fp8_weight_channel_calibrate_quantize", lambda: (rnd(4096, 4096),),
        lambda w: ops.absmax_quantize(w, codec="dtype", out_dtype=torch.float8_e4m3fn, **kw8), 2 * n, 3 * n, 3 * n)
    na = 8192 * 4096
    def act():
        x = torch.randn(1, 8192, 4096, generator=g, device=dev)
        x[..., torch.randperm(4096, generator=g, device=dev)[:41]] *= 20
        return (x.to(torch.bfloat16),)
    run("c2_fp8_activation_token_calibrate_quantize", act,
        lambda x: ops.absmax_quantize(x, codec="dtype", out_dtype=torch.float8_e4m3fn, **kw8), 2 * na, 3 * na, 3 * na)
    def c2_dq_args():
        return ops.absmax_quantize(act()[0], codec="dtype", out_dtype=torch.float8_e4m3fn, **kw8)
    run("c2_fp8_activation_dequantize", c2_dq_args,
        lambda q, sc: ops.dequantize(q, sc, None, scale_row_stride=1, out_dtype=torch.bfloat16, **kw8), 2 * na, 3 * na, 3 * na)
    nm = 14336 * 4096
    kwf = dict(qtype=ops.QFLOAT, bits=4, col_group=16)
    def nv(w):
        mn, mx = ops.minmax(w, w.shape[0], w.shape[1])
        gs = ops.generate_gparam(mn, mx)
        return ops.absmax_quantize(w, codec="fp4x2", global_scale=gs, **kwf) + (gs,)
    run("c3_nvfp4_amax_scales_quantize_pack", lambda: (rnd(14336, 4096),), nv, 2 * nm, 4.5625 * nm, 2.6 * nm)
    run("c3_nvfp4_unpack_dequantize", lambda: nv(rnd(4096, 14336)),
        lambda p, sc, gs: ops.dequantize(p, sc, None, scale_row_stride=14336 // 16, out_dtype=torch.bfloat16, codec="fp4x2", global_scale=gs, **kwf),
        2 * nm, 2.5625 * nm, 2.6 * nm)
    ns = 4096 * 11008
    def s24():
        w = rnd(4096, 11008)
        keep = ops.sparse24_mask(w)
        w = torch.where(keep, w, torch.zeros((), dtype=w.dtype, device=dev))
        q, _ = ops.absmax_quantize(w, qtype=ops.QFLOAT, bits=8, col_group=11008, codec="dtype", out_dtype=torch.float8_e4m3fn)
        return (q,)
    run("c4a_sparse24_compress_e4m3", s24, lambda q: ops.sparse24_compress(q), 2 * ns, 1.625 * ns, 1.7 * ns)
    def s24_dense():
        w = rnd(4096, 11008)
        w = torch.where(ops.sparse24_mask(w), w, torch.zeros((), dtype=w.dtype, device=dev))
        mn, mx = ops.minmax(w, 1, 11008)
        scale, _ = ops.calculate_qparams(mn, mx, qtype=ops.QFLOAT, bits=8, symmetric=True)
        return (w, scale.reshape(-1))
    # the whole of configuration 4a in one pass: pruned bf16 weight + per-channel scale in, kept e4m3 values + bitmask out
    run("c4a_fused_fp8_quantize_sparse24_compress", s24_dense, lambda w, sc: ops.quantize_fp8_sparse24(w, sc),
        2 * ns, 2.625 * ns, 2.7 * ns)
    def s24_packed():
        w, sc = s24_dense()
        return ops.quantize_fp8_sparse24(w, sc) + (sc,)
    run("c4a_fused_sparse24_decompress_fp8_dequantize", s24_packed,
        lambda v, b, sc: ops.sparse24_decompress_dequantize_fp8(v, b, sc, (4096, 11008)), 2 * ns, 2.625 * ns, 2.7 * ns)
    run("c4a_sparse24_decompress_e4m3", lambda: ops.sparse24_compress(s24()[0]),
        lambda v, b: ops.sparse24_decompress(v, b, (4096, 11008)), 2 * ns, 1.625 * ns, 1.7 * ns)
    def unstructured():
        w = rnd(4096, 4096)
        w[torch.rand(4096, 4096, generator=g, device=dev) < 0.5] = 0
        return (w,)
    run("c4b_bitmask_compress_bf16_50pct", unstructured, lambda w: ops._masked_compress(w, None, sync=False), 2 * n, (2 + 1 + 0.125) * n, 3.2 * n)
    run("c4b_bitmask_decompress_bf16_50pct", lambda: ops.bitmask_compress(unstructured()[0])[:2],
        lambda v, b: ops.bitmask_decompress(v, b, (4096, 4096)), 2 * n, (2 + 1 + 0.125) * n, 3.2 * n)
    return out


def copy_ceiling(dev, bytes_w, bytes_p, world):
    """What the PCIe copies of one end-to-end step cost on their own: the step's byte mix (weights in, packed out,
    packed in, weights out) as bare copies between page-locked host memory and the device, both directions at
    once on two streams, every rank doing the same at the same time.  Returned in the metric's unit (bf16 weight
    bytes through both directions per second, all ranks), so that e2e.value can be read against it."""
    import torch.distributed as dist

    chunk = 256 << 20
    host_a = torch.empty(chunk, dtype=torch.uint8, pin_memory=True)
    host_b = torch.empty(chunk, dtype=torch.uint8, pin_memory=True)
    dev_a = torch.empty(chunk, dtype=torch.uint8, device=dev)
    dev_b = torch.empty(chunk, dtype=torch.uint8, device=dev)
    s1, s2 = torch.cuda.Stream(dev), torch.cuda.Stream(dev)

    def run():
        for stream, dst, src, total in ((s1, dev_a, host_a, bytes_w + bytes_p), (s2, host_b, dev_b, bytes_p + bytes_w)):
            with torch.cuda.stream(stream):
                left = total
                while left > 0:
                    n = min(left, chunk)
                    dst[:n].copy_(src[:n], non_blocking=True)
                    left -= n
        s1.synchronize()
        s2.synchronize()

    run()
    if world > 1:
        dist.barrier()
    t0 = time.perf_counter()
    run()
    dt = torch.tensor([time.perf_counter() - t0], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(dt, op=dist.ReduceOp.MAX)
    return 2 * bytes_w * world / float(dt) / 1e9


def per_config_cpu(ct):
    """Seconds the reference's own functions take on this host for the stages behind each per_config row (all host
    threads, eager mode, seeded inputs of the named shapes; best of two, a single run for stages over half a second)."""
    from compressed_tensors.compressors.quantized_compressors.fp4_quantized import pack_fp4_to_uint8, unpack_fp4_from_uint8
    from compressed_tensors.compressors.quantized_compressors.pack_quantized import pack_to_int32, unpack_from_int32
    from compressed_tensors.compressors.sparse_compressors.sparse_24_bitmask import (get_24_bytemasks, sparse24_bitmask_compress,
                                                                                       sparse24_bitmask_decompress)
    from compressed_tensors.compressors.sparse_compressors.sparse_bitmask import bitmask_compress, bitmask_decompress
    from compressed_tensors.quantization import QuantizationArgs
    from compressed_tensors.quantization.lifecycle.forward import dequantize, quantize
    from compressed_tensors.quantization.utils.helpers import calculate_qparams, compute_dynamic_scales_and_zp, generate_gparam

    g = torch.Generator().manual_seed(SEED + 1)
    out = {}

    def timed(name, fn):
        t0 = time.perf_counter()
        res = fn()
        dt = time.perf_counter() - t0
        if dt < 0.5:
            t0 = time.perf_counter()
            res = fn()
            dt = min(dt, time.perf_counter() - t0)
        out[name] = dt
        return res

    def rnd(r, c, std=0.02):
        return (torch.randn(r, c, generator=g) * std).to(torch.bfloat16)

    with torch.no_grad():
        w = rnd(4096, 4096)
        a4 = QuantizationArgs(num_bits=4, symmetric=True, strategy="group", group_size=128)

        def c1():
            grouped = w.unflatten(-1, (-1, 128))
            s, z = calculate_qparams(grouped.amin(-1), grouped.amax(-1), a4)
            return pack_to_int32(quantize(w, s, z, a4, dtype=torch.int8), 4), s
        words, s4 = timed("c1_w4a16_calibrate_quantize_pack", c1)
        timed("c1_w4a16_unpack_dequantize", lambda: dequantize(unpack_from_int32(words, 4, w.shape), s4))
        a8 = QuantizationArgs(num_bits=8, type="float", symmetric=True, strategy="channel")

        def c2w():
            s, z = calculate_qparams(w.amin(-1, keepdim=True), w.amax(-1, keepdim=True), a8)
            return quantize(w, s, z, a8, dtype=torch.float8_e4m3fn)
        timed("c2_fp8_weight_channel_calibrate_quantize", c2w)
        x = torch.randn(1, 8192, 4096, generator=g)
        x[..., torch.randperm(4096, generator=g)[:41]] *= 20
        x = x.to(torch.bfloat16)
        at = QuantizationArgs(num_bits=8, type="float", symmetric=True, strategy="token", dynamic=True)

        def c2a():
            s, z = compute_dynamic_scales_and_zp(x, at, torch.nn.Identity())
            return quantize(x, s, z, at, dtype=torch.float8_e4m3fn), s
        xq, sx = timed("c2_fp8_activation_token_calibrate_quantize", c2a)
        timed("c2_fp8_activation_dequantize", lambda: dequantize(xq, sx, None, at))
        wn = rnd(14336, 4096)
        af = QuantizationArgs(num_bits=4, type="float", symmetric=True, strategy="tensor_group", group_size=16)

        def c3():
            mn, mx = torch.aminmax(wn)
            gs = generate_gparam(mn, mx)
            grouped = wn.unflatten(-1, (-1, 16))
            s, z = calculate_qparams(grouped.amin(-1), grouped.amax(-1), af, global_scale=gs)
            return pack_fp4_to_uint8(quantize(wn, s, z, af, global_scale=gs)), s, gs
        packed, sn, gs = timed("c3_nvfp4_amax_scales_quantize_pack", c3)
        timed("c3_nvfp4_unpack_dequantize",
              lambda: dequantize(unpack_fp4_from_uint8(packed, 14336, 4096), sn, global_scale=gs, dtype=torch.bfloat16))
        ws = rnd(4096, 11008)
        ws = torch.where(get_24_bytemasks(ws), ws, torch.zeros((), dtype=ws.dtype))
        s, z = calculate_qparams(ws.amin(-1, keepdim=True), ws.amax(-1, keepdim=True), a8)
        q = quantize(ws, s, z, a8, dtype=torch.float8_e4m3fn)
        vals, bm = timed("c4a_sparse24_compress_e4m3", lambda: sparse24_bitmask_compress(q))
        timed("c4a_fused_fp8_quantize_sparse24_compress",
              lambda: sparse24_bitmask_compress(quantize(ws, s, z, a8, dtype=torch.float8_e4m3fn)))
        timed("c4a_sparse24_decompress_e4m3", lambda: sparse24_bitmask_decompress(vals, bm, q.shape))
        timed("c4a_fused_sparse24_decompress_fp8_dequantize",
              lambda: dequantize(sparse24_bitmask_decompress(vals, bm, q.shape), s, None, a8, dtype=torch.bfloat16))
        wu = rnd(4096, 4096)
        wu[torch.rand(4096, 4096, generator=g) < 0.5] = 0
        v, b, _ = timed("c4b_bitmask_compress_bf16_50pct", lambda: bitmask_compress(wu))
        timed("c4b_bitmask_decompress_bf16_50pct", lambda: bitmask_decompress(v, b, wu.shape))
    return out


def standalone_ops_table(dev, peak, size=8192):
    """Device-timed throughput of the reference's operators as separate calls with given qparams (the building blocks the
    compressors and the calibration lifecycle call one by one) on a size x size bf16 tensor: quantize to packed words /
    int8 / e4m3 codes, fake_quantize, min/max per strategy, the stand-alone packers, whole-dimension Hadamard."""
    from compressed_tensors_b200 import ops

    out = {}
    run = op_timer(out, peak)
    g = torch.Generator(device=dev).manual_seed(SEED + 2)
    R = C = size
    n = R * C

    def rnd():
        return (torch.randn(R, C, generator=g, device=dev) * 0.02).to(torch.bfloat16)

    w0 = rnd()
    kw4 = dict(qtype=ops.QINT, bits=4, col_group=128, scale_row_stride=C // 128)
    mn, mx = ops.minmax(w0, 1, 128)
    s4, _ = ops.calculate_qparams(mn, mx, qtype=ops.QINT, bits=4, symmetric=True)
    s4a, z4a = ops.calculate_qparams(mn, mx, qtype=ops.QINT, bits=4, symmetric=False)
    kw8 = dict(qtype=ops.QINT, bits=8, col_group=C, scale_row_stride=1)
    mn, mx = ops.minmax(w0, 1, C)
    s8, _ = ops.calculate_qparams(mn, mx, qtype=ops.QINT, bits=8, symmetric=True)
    kwf = dict(qtype=ops.QFLOAT, bits=8, col_group=C, scale_row_stride=1)
    sf, _ = ops.calculate_qparams(mn, mx, qtype=ops.QFLOAT, bits=8, symmetric=True)
    kwb = dict(qtype=ops.QFLOAT, bits=8, col_group=128, row_group=128, scale_row_stride=C // 128)
    mn, mx = ops.minmax(w0, 128, 128)
    sb, _ = ops.calculate_qparams(mn, mx, qtype=ops.QFLOAT, bits=8, symmetric=True)
    one = lambda: (rnd(),)
    run("quantize_int4_g128_pack32", one, lambda w: ops.quantize(w, s4, None, codec="pack32", **kw4), 2 * n, 2.515625 * n, 2.6 * n)
    run("quantize_int4_g128_asym_pack32", one, lambda w: ops.quantize(w, s4a, z4a, codec="pack32", **kw4), 2 * n, 2.53 * n, 2.6 * n)
    run("quantize_int8_channel_codes", one, lambda w: ops.quantize(w, s8, None, out_dtype=torch.int8, **kw8), 2 * n, 3 * n, 3 * n)
    run("fake_quantize_int4_g128", one, lambda w: ops.fake_quantize(w, s4, None, out_dtype=torch.bfloat16, **kw4), 2 * n, 4 * n, 4 * n)
    run("fake_quantize_int8_channel", one, lambda w: ops.fake_quantize(w, s8, None, out_dtype=torch.bfloat16, **kw8), 2 * n, 4 * n, 4 * n)
    run("quantize_fp8_channel", one, lambda w: ops.quantize(w, sf, None, out_dtype=torch.float8_e4m3fn, **kwf), 2 * n, 3 * n, 3 * n)
    run("quantize_fp8_block128x128", one, lambda w: ops.quantize(w, sb, None, out_dtype=torch.float8_e4m3fn, **kwb), 2 * n, 3 * n, 3 * n)
    run("fake_quantize_fp8_block128x128", one, lambda w: ops.fake_quantize(w, sb, None, out_dtype=torch.bfloat16, **kwb), 2 * n, 4 * n, 4 * n)
    s8f, sff = s8.float(), sf.float()
    run("quantize_int8_channel_fp32_scale", one, lambda w: ops.quantize(w, s8f, None, out_dtype=torch.int8, **kw8), 2 * n, 3 * n, 3 * n)
    run("quantize_fp8_channel_fp32_scale", one, lambda w: ops.quantize(w, sff, None, out_dtype=torch.float8_e4m3fn, **kwf), 2 * n, 3 * n, 3 * n)
    run("fake_quantize_fp8_channel_fp32_scale", one, lambda w: ops.fake_quantize(w, sff, None, out_dtype=torch.bfloat16, **kwf), 2 * n, 4 * n, 4 * n)
    run("dequantize_int4_g128_pack32", lambda: (ops.quantize(rnd(), s4, None, codec="pack32", **kw4),),
        lambda p: ops.dequantize(p, s4, None, out_dtype=torch.bfloat16, codec="pack32", cols=C, **kw4), 2 * n, 2.515625 * n, 2.6 * n)
    run("dequantize_int4_g128_asym_pack32", lambda: (ops.quantize(rnd(), s4a, z4a, codec="pack32", **kw4),),
        lambda p: ops.dequantize(p, s4a, z4a, out_dtype=torch.bfloat16, codec="pack32", cols=C, **kw4), 2 * n, 2.53 * n, 2.6 * n)
    run("dequantize_int8_channel", lambda: (ops.quantize(rnd(), s8, None, out_dtype=torch.int8, **kw8),),
        lambda q: ops.dequantize(q, s8, None, out_dtype=torch.bfloat16, **kw8), 2 * n, 3 * n, 3 * n)
    run("dequantize_fp8_channel", lambda: (ops.quantize(rnd(), sf, None, out_dtype=torch.float8_e4m3fn, **kwf),),
        lambda q: ops.dequantize(q, sf, None, out_dtype=torch.bfloat16, **kwf), 2 * n, 3 * n, 3 * n)
    run("dequantize_fp8_block128x128", lambda: (ops.quantize(rnd(), sb, None, out_dtype=torch.float8_e4m3fn, **kwb),),
        lambda q: ops.dequantize(q, sb, None, out_dtype=torch.bfloat16, **kwb), 2 * n, 3 * n, 3 * n)
    gi = (torch.arange(C, device=dev, dtype=torch.int32) // 128)[torch.randperm(C, generator=g, device=dev)].contiguous()
    run("quantize_int4_g128_actorder_codes", one, lambda w: ops.quantize(w, s4, None, out_dtype=torch.int8, g_idx=gi, **kw4), 2 * n, 3 * n, 3 * n)
    run("dequantize_int4_g128_actorder_pack32", lambda: (ops.quantize(rnd(), s4, None, codec="pack32", g_idx=gi, **kw4),),
        lambda p: ops.dequantize(p, s4, None, out_dtype=torch.bfloat16, codec="pack32", cols=C, g_idx=gi, **kw4), 2 * n, 2.515625 * n, 2.6 * n)
    nt = 8192 * 4096
    tok = lambda: (torch.randn(1, 8192, 4096, generator=g, device=dev).to(torch.bfloat16),)
    from compressed_tensors_b200.quantization import QuantizationArgs, forward_quantize
    for label, a in (("int8", QuantizationArgs(num_bits=8, symmetric=True, strategy="token", dynamic=True)),
                     ("fp8", QuantizationArgs(num_bits=8, type="float", symmetric=True, strategy="token", dynamic=True))):
        run(f"forward_quantize_dynamic_token_{label}_8192x4096", tok, lambda x, a=a: forward_quantize(None, x, "input", a), 2 * nt, 4 * nt, 4 * nt)
    ga = QuantizationArgs(num_bits=8, type="float", symmetric=True, strategy="group", group_size=128, dynamic=True)
    run("forward_quantize_dynamic_group128_fp8_8192x4096", tok, lambda x: forward_quantize(None, x, "input", ga), 2 * nt, 4 * nt, 4 * nt)
    run("minmax_group128", one, lambda w: ops.minmax(w, 1, 128), 2 * n, 2 * n, 2 * n)
    run("minmax_channel", one, lambda w: ops.minmax(w, 1, C), 2 * n, 2 * n, 2 * n)
    run("minmax_block128x128", one, lambda w: ops.minmax(w, 128, 128), 2 * n, 2 * n, 2 * n)
    run("minmax_tensor", one, lambda w: ops.minmax(w, R, C), 2 * n, 2 * n, 2 * n)
    codes = lambda: (ops.quantize(rnd(), s4, None, out_dtype=torch.int8, **kw4),)
    run("pack_to_int32_4bit", codes, lambda q: ops.pack_int32(q, 4), 2 * n, 1.5 * n, 1.5 * n)
    run("unpack_from_int32_4bit", lambda: (ops.pack_int32(codes()[0], 4),), lambda p: ops.unpack_int32(p, 4, (R, C)), 2 * n, 1.5 * n, 1.5 * n)
    masks = lambda: (rnd() > 0,)
    run("pack_bitmasks", masks, lambda m: ops.pack_bitmasks(m), 2 * n, 1.125 * n, 1.125 * n)
    run("unpack_bitmasks", lambda: (ops.pack_bitmasks(masks()[0]),), lambda p: ops.unpack_bitmasks(p, [R, C]), 2 * n, 1.125 * n, 1.125 * n)
    fp4 = lambda: (ops.unpack_fp4(torch.randint(0, 256, (R, C // 2), device=dev, dtype=torch.uint8, generator=g), R, C),)
    run("pack_fp4_to_uint8", fp4, lambda q: ops.pack_fp4(q), 2 * n, 2.5 * n, 2.5 * n)
    run("unpack_fp4_from_uint8", lambda: (ops.pack_fp4(fp4()[0]),), lambda p: ops.unpack_fp4(p, R, C), 2 * n, 2.5 * n, 2.5 * n)
    run("get_24_bytemasks", one, lambda w: ops.sparse24_mask(w), 2 * n, 3 * n, 3 * n)
    for hn in (128, 4096):
        sg = (torch.randint(0, 2, (hn,), device=dev, generator=g) * 2 - 1).to(torch.int8)
        for side, tag in ((0, "weight_input"), (1, "weight_output")):
            for prec, ptag in ((torch.float32, "f32"), (torch.float64, "f64")):
                run(f"hadamard_{tag}_n{hn}_{ptag}", one, lambda w, side=side, prec=prec, hn=hn, sg=sg: ops.hadamard(w, hn, signs=sg, side=side, precision=prec),
                    2 * n, 4 * n, 4 * n)
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--precision", default="tc", choices=["f64", "f32", "tc"],
                    help="Hadamard rotation: float64 butterfly (bit-identical to the reference), float32 butterfly, or tcgen05 tensor cores with fp32 accumulators")
    ap.add_argument("--layers", type=int, default=32, help="decoder layers of the model (32 = Llama-3-8B)")
    ap.add_argument("--no-reuse-buffers", action="store_true",
                    help="every compress_model / decompress_model call allocates fresh outputs and re-walks the module tree (the default of ModelCompressor)")
    ap.add_argument("--no-copy-ceiling", action="store_true", help="skip timing bare pinned copies with the round trip's byte mix")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-per-config", action="store_true", help="skip the C1-C4 per-scheme table")
    ap.add_argument("--no-other-modes", action="store_true", help="skip timing the other rotation arithmetics")
    ap.add_argument("--per-config-only", action="store_true",
                    help="time the C1-C4 per-scheme table alone, print it and exit (1 GPU; the small case for profiling one of its kernels)")
    ap.add_argument("--standalone-ops", action="store_true",
                    help="time the operators as separate calls on an 8192 x 8192 tensor, print that table alone and exit (1 GPU)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    quiet_stdout()
    if args.impl == "reference":
        return run_reference(args)

    import torch.distributed as dist
    from compressed_tensors_b200 import _lib, ops, parallel

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    if args.per_config_only:
        if rank == 0:
            emit({"per_config": per_config_table(dev, peaks()[0]), "peak_gbs": peaks()[0],
                  "timing": "CUDA events over CUDA-graph replays, rotating inputs larger than 2x L2"})
        if world > 1:
            dist.destroy_process_group()
        return
    if args.standalone_ops:
        if rank == 0:
            emit({"standalone_ops": standalone_ops_table(dev, peaks()[0]), "tensor": "8192x8192 bf16",
                  "peak_gbs": peaks()[0], "timing": "CUDA events over CUDA-graph replays, rotating inputs larger than L2"})
        if world > 1:
            dist.destroy_process_group()
        return

    import compressed_tensors_b200 as ctb
    import compressed_tensors_b200.compressors, compressed_tensors_b200.quantization, compressed_tensors_b200.transform  # noqa: F401
    from compressed_tensors_b200.compressors import ModelCompressor

    shape = parallel.LLAMA3_8B
    shapes = parallel.linear_shapes(shape)
    my_layers = parallel.partition_layers(args.layers, world, rank)
    weights = make_weights(my_layers, dev, shapes)
    total_elems = sum(o * i for _, o, i in shapes) * args.layers
    rank_elems = sum(w.numel() for w in weights)
    tcfg, qcfg = configs(ctb)
    rotation = {"f64": "exact", "f32": "float32", "tc": "tensor"}[args.precision]

    def new_compressor(**kw):
        return ModelCompressor(quantization_config=qcfg.model_copy(deep=True), transform_config=tcfg, rotation_precision=rotation, **kw)

    # ---- device-resident: the module tree lives on the GPU, both calls leave their results there
    model = build_model(my_layers, shapes, [w.clone() for w in weights])
    ctb.quantization.apply_quantization_config(model, qcfg)
    mc = new_compressor(reuse_buffers=not args.no_reuse_buffers)
    mc.engine.record_kernel_times = True
    stream = torch.cuda.current_stream()

    def compress():
        if getattr(model, "transform_config", None) is not None:
            del model.transform_config  # the dequantized weights of the last step are this step's fresh, un-rotated model
        mc.compress_model(model)

    def decompress():
        mc.decompress_model(model)

    def step():
        compress()
        decompress()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        step()
    barrier()
    mc.engine.kernel_times.clear()
    launches0 = mc.engine.launches
    sampler = ClockSampler(local) if rank == 0 else None
    t = time_region(step, args.steps, stream)
    barrier()
    clocks = sampler.stop() if sampler else None
    launches = mc.engine.launches - launches0
    # duration of the two kernels themselves inside that timed region (CUDA events recorded around each launch)
    tc = sum(a.elapsed_time(b) for kind, a, b in mc.engine.kernel_times if kind == "compress") / 1e3
    td = sum(a.elapsed_time(b) for kind, a, b in mc.engine.kernel_times if kind == "decompress") / 1e3
    mc.engine.record_kernel_times = False
    mc.engine.kernel_times.clear()
    # the same steps through the general path of ModelCompressor (no recorded cycle: every call walks the module tree,
    # allocates its outputs and re-installs the parameters), for the record
    tg = 0.0
    if not args.no_reuse_buffers:
        mc_general = new_compressor()

        def general_step():
            if getattr(model, "transform_config", None) is not None:
                del model.transform_config
            mc_general.compress_model(model)
            mc_general.decompress_model(model)

        for _ in range(2):
            general_step()
        barrier()
        tg = time_region(general_step, max(3, min(args.steps, 5)), stream) / max(3, min(args.steps, 5))
        del mc_general
    times = torch.tensor([t, tc, td, tg], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    t, tc, td, tg = (float(v) for v in times.cpu())

    # ---- end to end: the module tree lives in page-locked HOST memory; copies in both directions are inside the timed region
    e2e = None
    if not args.no_e2e:
        host_w = [torch.empty(w.shape, dtype=w.dtype, pin_memory=True).copy_(w) for w in weights]
        torch.cuda.synchronize()
        hmodel = build_model(my_layers, shapes, host_w)
        ctb.quantization.apply_quantization_config(hmodel, qcfg)
        hmc = new_compressor()
        del host_w

        def trip():
            if getattr(hmodel, "transform_config", None) is not None:
                del hmodel.transform_config
            with hmc.pipelined():
                hmc.compress_model(hmodel)
                hmc.decompress_model(hmodel)

        first = {n: p.data.clone() for n, p in list(hmodel.named_parameters())[:len(shapes)]}
        trip()
        # the restored host weights of the first layer must be what the device path produces from the same weights
        check = build_model(my_layers[:1], shapes, [v.to(dev) for v in first.values()])
        ctb.quantization.apply_quantization_config(check, qcfg)
        cmc = new_compressor()
        cmc.compress_model(check)
        cmc.decompress_model(check)
        torch.cuda.synchronize()
        got = {n: p.data for n, p in hmodel.named_parameters() if n.endswith(".weight") and n.startswith("model.layers.0.")}
        want = {n: p.data.cpu() for n, p in check.named_parameters() if n.endswith(".weight")}
        for n, v in want.items():
            assert torch.equal(got[n], v), f"end-to-end result differs from the device path: {n}"
        del check, cmc, first, got, want
        # more untimed trips, until every page-locked block of a trip comes out of the staging pool (the blocks of the
        # trip before are released while this trip's copies still read them: it takes two generations)
        from compressed_tensors_b200 import pinned
        for _ in range(6):
            before = pinned.pool().allocations
            trip()
            if pinned.pool().allocations == before:
                break
        barrier()
        bytes_w = 2 * rank_elems
        bytes_p = rank_elems // 2 + 2 * (rank_elems // 128)
        k = max(1, min(args.steps, 3))
        t0 = time.perf_counter()
        for _ in range(k):
            trip()
        te = torch.tensor([(time.perf_counter() - t0) / k], dtype=torch.float64, device=dev)
        # the same trip without letting the two calls overlap (each call waits for its own results); all ranks start
        # together, so that every rank sees the host-memory and PCIe contention of the others
        barrier()
        t0 = time.perf_counter()
        if getattr(hmodel, "transform_config", None) is not None:
            del hmodel.transform_config
        hmc.compress_model(hmodel)
        hmc.decompress_model(hmodel)
        ts = torch.tensor([time.perf_counter() - t0], dtype=torch.float64, device=dev)
        ceiling = None if args.no_copy_ceiling else copy_ceiling(dev, bytes_w, bytes_p, world)
        if world > 1:
            dist.all_reduce(te, op=dist.ReduceOp.MAX)
            dist.all_reduce(ts, op=dist.ReduceOp.MAX)
        e2e = {"value": 2 * 2 * total_elems / float(te) / 1e9, "unit": UNIT,
               "h2d_bytes_per_step": bytes_w + bytes_p, "d2h_bytes_per_step": bytes_p + bytes_w,
               "ms_per_step": float(te) * 1e3, "bytes_are": "per rank",
               "sequential_value": 2 * 2 * total_elems / float(ts) / 1e9,
               "copy_ceiling_gbs": ceiling,
               "path": "ModelCompressor.compress_model + ModelCompressor.decompress_model on a module tree in page-locked host memory, "
                       "inside ModelCompressor.pipelined(): host -> device -> fused kernels -> host, one decoder layer per pipeline step; "
                       "sequential_value = the same two calls without pipelined()"}
        del hmodel, hmc

    if rank == 0:
        peak, peak_kind = peaks()
        ms = t / args.steps * 1e3
        # dominant kernel: the fused rotate+calibrate+quantize+pack launch of compress_model.
        # per-rank algorithmic bytes of one compress pass / average device time of that launch
        achieved = ALG_BYTES_PER_ELEM * rank_elems / (tc / args.steps) / 1e9
        cfg = workload_config(args.layers, world, args.precision)
        cfg.update({"tensors_per_rank": len(weights), "api": "ModelCompressor.compress_model / decompress_model on a CUDA-resident module tree",
                    "reuse_buffers": not args.no_reuse_buffers,
                    "one_grid_per_shard": launches == 2 * args.steps})
        out = {
            "metric": METRIC, "value": 2 * 2 * total_elems / (t / args.steps) / 1e9, "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": cfg,
            "general_path": None if tg == 0.0 else {"value": 2 * 2 * total_elems / tg / 1e9, "ms_per_step": tg * 1e3,
                                                    "note": "reuse_buffers=False: host-bound (one Python walk over the module tree per call)"},
            "kernel_compress_gbs": 2 * rank_elems * world / (tc / args.steps) / 1e9, "kernel_decompress_gbs": 2 * rank_elems * world / (td / args.steps) / 1e9,
            "kernel_ms_per_step": (tc + td) / args.steps * 1e3,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": (NCU_TRAFFIC_BYTES_PER_ELEM * rank_elems) if args.precision == "tc" else None,
                         "traffic_source": "ncu capture of the 2-layer case scaled by elements per launch", "kernel": "rotquant128_tc_kernel" if args.precision == "tc" else "rotquant128_kernel", "peak_kind": peak_kind,
                         "timed": "CUDA events around the launch, on its stream, inside the timed region",
                         "decompress_frac": ALG_BYTES_PER_ELEM * rank_elems / (td / args.steps) / 1e9 / peak},
            "clocks": clocks, "gpu_launches": int(launches), "e2e": e2e,
        }
        if world == 1 and not args.no_other_modes:
            # the same compress pass with the other two rotation arithmetics, for the record (kernel time only)
            modes = {}
            for tag, prec in (("f64", torch.float64), ("f32", torch.float32), ("tc", ops.ROT_TENSOR)):
                if tag == args.precision:
                    continue
                alt = parallel.ShardCodec(weights, group_size=128, hadamard_n=128, signs=make_signs().to(dev), precision=prec, use_graphs=False)
                alt.compress()
                torch.cuda.synchronize()
                ta = time_region(alt.compress, 3, stream) / 3
                modes[tag] = {"compress_gbs": round(2 * total_elems / ta / 1e9, 1), "frac": round(ALG_BYTES_PER_ELEM * total_elems / ta / 1e9 / peak, 3)}
                del alt
            out["other_rotation_modes"] = modes
            out["other_schemes"] = {
                "fp8_channel_float_quantized": scheme_shard_leg("fp8", ctb, ModelCompressor, weights, my_layers, shapes, dev, peak),
                "nvfp4_pack_quantized": scheme_shard_leg("nvfp4", ctb, ModelCompressor, weights, my_layers, shapes, dev, peak)}
        arm = None
        if world == 1 and not args.no_cpu_baseline:
            arm = CpuArm()
        if world == 1 and not args.no_per_config:
            del model, mc, weights
            torch.cuda.empty_cache()
            out["per_config"] = per_config_table(dev, peak)
            if arm is not None and arm.kind == "reference":
                for name, sec in per_config_cpu(arm.ct).items():
                    if name in out["per_config"]:
                        out["per_config"][name]["cpu_reference_ms"] = round(sec * 1e3, 1)
                        out["per_config"][name]["cpu_reference_dense_gbs"] = round(out["per_config"][name]["dense_gbs"] * out["per_config"][name]["us"] / (sec * 1e6), 3)
        if arm is not None:
            dt, val = arm.time(2, 1)
            out["cpu_baseline"] = {"value": val, "unit": UNIT, "cores": arm.cores, "kind": arm.kind, "sample": SAMPLE_TEXT + ", 2 passes"}
        emit(out)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
