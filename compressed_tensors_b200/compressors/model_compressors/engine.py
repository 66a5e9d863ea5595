"""The machinery under ModelCompressor: whole-model compress / decompress as a few large grids and a
copy pipeline instead of the reference's tensor-by-tensor walk
(compressors/model_compressors/model_compressor.py:453-617 driving quantized_compressors/base.py:69-134
and sparse_compressors/base.py:66-107 once per module).

A *job* is one module's parameters.  Jobs whose weights already live on a GPU are processed where they are,
all at once.  Jobs whose weights live in host memory are cut into *steps* of a few hundred megabytes and
streamed: copy-in, kernels and copy-out of consecutive steps run on three streams, so both PCIe directions
and the GPU work at the same time, nothing synchronises per tensor, and results land in page-locked host
memory.  Inside a step, every weight of a scheme that has a whole-shard entry point (W4A16 group 128 with
or without the block-128 Hadamard rotation in front, and its unpack + dequantize) goes through ONE launch;
everything else calls the per-tensor compressor on the device tensors of the step.

The results are those of the per-tensor walk: the batched kernels are the per-tensor kernels run over a
table, and the per-tensor compressors are the registered ones.
"""
import contextlib
import ctypes
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch
from torch import Tensor

from ... import _lib as L
from ... import ops
from ...pinned import pool as pinned_pool
from ...config import CompressionFormat
from ...quantization.quant_args import QuantizationArgs, QuantizationStrategy, QuantizationType
from ...quantization.utils.helpers import calculate_qparams, generate_gparam, is_fp4

__all__ = ["Job", "CodecEngine", "minmax_qparams", "is_w4a16_g128", "STEP_BYTES"]

STEP_BYTES = 256 << 20   # host-resident work is streamed in steps of about this many bytes on the bus
INFLIGHT_FRACTION = 0.4  # of the device memory that is free when a pass starts: bound on the buffers of steps in flight
_ALIGN = 256

# parameters a quantization compressor reads next to the weight
_QPARAMS = ("weight_scale", "weight_zero_point", "weight_g_idx", "weight_global_scale")


def is_w4a16_g128(args: Optional[QuantizationArgs]) -> bool:
    """True for the scheme the whole-shard int4 entry points are built for: symmetric int4, group 128, static."""
    return (args is not None and args.type == QuantizationType.INT and args.num_bits == 4 and args.symmetric
            and args.strategy == QuantizationStrategy.GROUP.value and args.group_size == 128 and not args.dynamic
            and args.actorder is None)


@torch.no_grad()
def minmax_qparams(weight: Tensor, args: QuantizationArgs) -> Dict[str, Tensor]:
    """Min-max calibration of one weight on its device: `weight_scale`, `weight_zero_point` and, for NVFP4,
    `weight_global_scale`, shaped as quantization/lifecycle/initialize.py:155-280 shapes them
    (quantization/utils/helpers.py:67-146 calculate_qparams over the strategy's reduction)."""
    rows, cols = weight.shape
    out: Dict[str, Tensor] = {}
    gs = None
    strategy = QuantizationStrategy(args.strategy)
    if strategy == QuantizationStrategy.TENSOR_GROUP:
        mn, mx = ops.minmax(weight, rows, cols)
        gs = generate_gparam(mn.reshape(()), mx.reshape(()))
        out["weight_global_scale"] = gs
    if strategy in (QuantizationStrategy.GROUP, QuantizationStrategy.TENSOR_GROUP):
        mn, mx = ops.minmax(weight, 1, args.group_size)
    elif strategy == QuantizationStrategy.CHANNEL:
        mn, mx = ops.minmax(weight, 1, cols)
    elif strategy == QuantizationStrategy.TENSOR:
        mn, mx = ops.minmax(weight, rows, cols)
        mn, mx = mn.reshape(()), mx.reshape(())
    elif strategy == QuantizationStrategy.BLOCK:
        bh, bw = args.block_structure
        mn, mx = ops.minmax(weight, bh, bw)
    else:
        raise NotImplementedError(f"weight calibration for strategy {args.strategy}")
    scale, zp = calculate_qparams(mn, mx, args, global_scale=gs if is_fp4(args) else None)
    out["weight_scale"], out["weight_zero_point"] = scale, zp
    return out


@dataclass
class Job:
    """One module's parameters on their way through a compressor."""

    prefix: str
    state: Dict[str, Tensor]                    # local parameter name -> tensor, where the caller keeps it
    scheme: object = None                       # QuantizationScheme or None
    compressor: object = None                   # the quantization compressor of the module's format, or None
    sparse: bool = False                        # the module is a target of the sparsity compressor
    transforms: Sequence = ()                   # weight-side transforms still to be fused (compress only)
    kind: str = "generic"
    shape: Optional[Tuple[int, int]] = None     # dense weight shape where it is known without reading a tensor
    # results; parameters that pass through unchanged are not repeated in any of them
    out: Dict[str, Tensor] = field(default_factory=dict)         # what compress_weight / decompress_weight returned
    qparams: Dict[str, Tensor] = field(default_factory=dict)     # scales the pass calibrated itself (fused rotation)
    sparse_out: Dict[str, Tensor] = field(default_factory=dict)  # the sparsity compressor's parameters (replace `weight`)
    quantized: bool = False                                      # compress_weight ran: `out` stands for `weight`

    def results(self):
        """(dict, name, tensor) over everything the pass produced."""
        for d in (self.out, self.qparams, self.sparse_out):
            for name, value in list(d.items()):
                yield d, name, value


def _nbytes(t: Tensor) -> int:
    return t.numel() * t.element_size()


def _up(n: int) -> int:
    return (n + _ALIGN - 1) // _ALIGN * _ALIGN


class _Arena:
    """A buffer handing out 256-byte aligned views: one allocation per step and side instead of one per tensor, and
    one contiguous span for the tensor map of the tensor-core kernel."""

    def __init__(self, nbytes: int, device=None, pinned: bool = False):
        if pinned:
            self.buf = pinned_pool().take(nbytes)
        else:
            self.buf = torch.empty(max(nbytes, 1), dtype=torch.uint8, device=device)
        self.off = 0
        self._typed: Dict[torch.dtype, Tensor] = {}

    def take(self, shape, dtype: torch.dtype) -> Tensor:
        """A contiguous view of `shape` and `dtype` at the next aligned offset."""
        item = _ITEMSIZE[dtype]
        typed = self._typed.get(dtype)
        if typed is None:
            typed = self._typed[dtype] = self.buf.view(dtype) if self.buf.numel() % item == 0 else self.buf[: self.buf.numel() // item * item].view(dtype)
        shape = tuple(int(s) for s in shape)
        n, strides = 1, []
        for d in reversed(shape):
            strides.append(n)
            n *= d
        view = typed.as_strided(shape, tuple(reversed(strides)), self.off // item)
        self.off += _up(n * item)
        return view


_ITEMSIZE = {torch.bfloat16: 2, torch.float16: 2, torch.float32: 4, torch.float64: 8, torch.int8: 1, torch.uint8: 1,
             torch.bool: 1, torch.int16: 2, torch.int32: 4, torch.int64: 8, torch.float8_e4m3fn: 1}


def _table(ins: List[Tensor], outs: List[Tensor], scales: List[Tensor], shapes: List[Tuple[int, int]]):
    """ctb_tensor_ref[n] as a numpy array (five int64 per entry: in, out, scale, rows, cols)."""
    n = len(ins)
    t = np.empty((n, 5), dtype=np.int64)
    t[:, 0] = [x.data_ptr() for x in ins]
    t[:, 1] = [x.data_ptr() for x in outs]
    t[:, 2] = [x.data_ptr() for x in scales]
    t[:, 3:5] = shapes
    return t


def _table_ptr(t: np.ndarray):
    return ctypes.cast(t.ctypes.data, ctypes.POINTER(L.TensorRef))


def _prod(shape) -> int:
    n = 1
    for d in shape:
        n *= int(d)
    return n


_PLANNED_KINDS = ("rotq4", "q4", "dq4", "q8c", "dq8c", "q4f", "dq4f")  # outputs known without running the step


class _Step:
    """A few hundred megabytes of one pass over host-resident jobs: upload, kernels, download."""

    def __init__(self, direction: str, jobs: List[Job], dev: torch.device, work, sparse_compress, need: int):
        self.direction, self.jobs, self.dev, self.work, self.sparse_compress, self.need = direction, jobs, dev, work, sparse_compress, need
        self.feeds: List[Dict[str, Tensor]] = []
        self.reads: set = set()        # host storages the step uploads
        self.writes: int = 0           # host storage its planned results live in
        self.planned: list = []        # (job, in qparams?, name, host tensor) for results created ahead of the run
        self.submitted = False
        self.successor_submitted = False


class CodecEngine:
    """Runs lists of jobs.  One engine per ModelCompressor; streams are created per device on first use."""

    def __init__(self, rotation_precision=torch.float64):
        self.rotation_precision = rotation_precision
        self._streams: Dict[Tuple[int, str], Tuple[torch.cuda.Stream, ...]] = {}
        self._status: Dict[int, Tensor] = {}
        self._signs: Dict[Tuple[int, int], Tuple[object, Tensor]] = {}
        # host storage -> event after which its bytes are valid (results still on their way while `deferred`)
        self._host_ready: Dict[int, torch.cuda.Event] = {}
        self._tail: List[torch.cuda.Event] = []
        self._queue: List[_Step] = []                 # planned, not yet submitted
        self._producer: Dict[int, _Step] = {}         # host storage -> the planned step that fills it
        self._last_submitted: Dict[str, _Step] = {}
        self._eager_head: Dict[str, int] = {}         # steps of a pass submitted ahead of the drain (deferred mode)
        self._inflight: Dict[int, List[Tuple[torch.cuda.Event, int]]] = {}
        self._budget: Dict[int, float] = {}
        self.deferred = False
        self.launches = 0
        self.fuse_sparse24 = False  # set by the owner when its sparsity compressor is sparse-24-bitmask
        # measurement hook: with record_kernel_times set, every whole-shard launch is bracketed by two CUDA events
        # on its stream and (kind, start, end) is appended to kernel_times
        self.record_kernel_times = False
        self.kernel_times: List[Tuple[str, torch.cuda.Event, torch.cuda.Event]] = []

    # ------------------------------------------------------------------ plumbing
    def _get_streams(self, dev: torch.device, role: str):
        """Copy-in, kernel and copy-out stream of `dev`, shared by both directions: copies of one direction execute
        in the order they were submitted whatever stream they are on, so more streams would buy nothing."""
        key = (dev.index, "")
        if key not in self._streams:
            self._streams[key] = tuple(torch.cuda.Stream(dev) for _ in range(3))
        return self._streams[key]

    def _signs_on(self, transform, dev: torch.device) -> Tensor:
        """The +-1 diagonal of a Hadamard transform on `dev`, copied over once: a copy from pageable host memory makes
        the host wait for the stream, which would tie the enqueueing of every pipeline step to the GPU's pace."""
        key = (id(transform), dev.index)
        hit = self._signs.get(key)
        if hit is None or hit[0] is not transform:
            hit = self._signs[key] = (transform, transform._signs.to(dev))
        return hit[1]

    def _status_word(self, dev: torch.device) -> Tensor:
        """The word a kernel of `dev` writes when one of its bounded waits gives up.  It lives in page-locked host
        memory that the device writes over the bus: reading it needs no copy, which on a busy pipeline would queue
        behind the large transfers of its direction and hold up the stream it was issued on."""
        if dev.index not in self._status:
            self._status[dev.index] = torch.zeros(1, dtype=torch.int32).pin_memory()
        return self._status[dev.index]

    @contextlib.contextmanager
    def _timed(self, kind: str, dev: torch.device):
        if not self.record_kernel_times:
            yield
            return
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(torch.cuda.current_stream(dev))
        yield
        b.record(torch.cuda.current_stream(dev))
        self.kernel_times.append((kind, a, b))

    def _check_status(self, wait: bool = False) -> None:
        """Raise for a time-out that a launch reported.  Without `wait` this sees what has been written so far; callers
        that need the verdict of everything enqueued synchronise first."""
        for idx, word in self._status.items():
            if int(word[0]) != 0:
                word.zero_()
                raise TimeoutError(f"a bounded wait inside the tensor-core rotation kernel gave up on cuda:{idx}; "
                                   "the outputs of that compress pass are incomplete")

    def finish(self) -> None:
        """Wait for everything this engine has put in flight, and turn a device-side time-out into an exception."""
        self._drain()
        for ev in self._tail:
            ev.synchronize()
        self._tail.clear()
        self._host_ready.clear()
        self._producer.clear()
        self._last_submitted.clear()
        self._eager_head.clear()
        self._inflight.clear()
        self._budget.clear()
        self._check_status(wait=True)
        if pinned_pool().has_parked():
            # Staging blocks whose tensors died may be handed out again once nothing queued can still touch them: the
            # waits above cover this engine's own copies; a device-wide wait covers copies the caller issued itself.
            torch.cuda.synchronize()
            pinned_pool().settle()

    # ------------------------------------------------------------------ compress
    def classify_compress(self, job: Job) -> None:
        job.kind = "generic"
        w = job.state.get("weight")
        if w is None or job.compressor is None or job.scheme is None or job.scheme.weights is None or w.ndim != 2:
            return
        args = job.scheme.weights
        fmt = getattr(job.compressor, "_format_name", None)
        rows, cols = w.shape
        if self._is_fp8_channel(job, fmt, args, rows, cols) and w.dtype == torch.bfloat16 and not job.transforms:
            zp = job.state.get("weight_zero_point")
            if zp is None or (zp.numel() == rows and zp.dtype in L.DT):
                job.kind = "q8c"
            return
        if self._is_nvfp4(job, fmt, args, rows, cols) and w.dtype == torch.bfloat16 and not job.transforms:
            zp, s = job.state.get("weight_zero_point"), job.state["weight_scale"]
            if zp is None or (tuple(zp.shape) == tuple(s.shape) and zp.dtype in L.DT):
                job.kind = "q4f"
            return
        if fmt != CompressionFormat.pack_quantized.value or not is_w4a16_g128(args) or w.dtype != torch.bfloat16 or cols % 128:
            return
        if job.sparse and "weight" in job.compressor.compression_param_names:
            return
        if job.transforms:
            if len(job.transforms) == 1 and _fusable_rotation(job.transforms[0]):
                if self.rotation_precision != ops.ROT_TENSOR or (rows * cols) % (128 * 128) == 0:
                    job.kind = "rotq4"
            return
        s = job.state.get("weight_scale")
        if (s is not None and s.dtype == torch.bfloat16 and tuple(s.shape) == (rows, cols // 128)
                and job.state.get("weight_g_idx") is None):
            job.kind = "q4"

    @staticmethod
    def _is_fp8_channel(job: Job, fmt, args, rows: int, cols: int) -> bool:
        """Static per-output-channel FP8 of a 2-D weight through the float-quantized compressor, not stacked with a
        sparsity compressor: what the whole-shard FP8 entry points take."""
        s = job.state.get("weight_scale")
        return (fmt == CompressionFormat.float_quantized.value and args is not None and args.type == QuantizationType.FLOAT
                and args.num_bits == 8 and args.strategy == QuantizationStrategy.CHANNEL and not args.dynamic
                and not job.sparse and cols % 8 == 0 and s is not None and s.dtype == torch.bfloat16 and s.numel() == rows
                and job.state.get("weight_g_idx") is None and job.state.get("weight_global_scale") is None)

    @staticmethod
    def _is_nvfp4(job: Job, fmt, args, rows: int, cols: int) -> bool:
        """NVFP4 (e2m1 codes, e4m3 group-16 scales, fp32 global scale) of a 2-D weight through the nvfp4-pack-quantized
        compressor, not stacked with a sparsity compressor: what the whole-shard NVFP4 entry points take."""
        s, gs = job.state.get("weight_scale"), job.state.get("weight_global_scale")
        return (fmt == CompressionFormat.nvfp4_pack_quantized.value and args is not None and args.type == QuantizationType.FLOAT
                and args.num_bits == 4 and args.strategy == QuantizationStrategy.TENSOR_GROUP and args.group_size == 16
                and not args.dynamic and not job.sparse and cols % 16 == 0 and s is not None and s.dtype == torch.float8_e4m3fn
                and tuple(s.shape) == (rows, cols // 16) and gs is not None and gs.dtype == torch.float32 and gs.numel() == 1
                and job.state.get("weight_g_idx") is None)

    def _compress_on_device(self, jobs: List[Job], dev: torch.device) -> None:
        """All jobs hold device tensors of `dev`; the current stream is the one to launch on.  Fills job.out
        with device tensors."""
        rot = [j for j in jobs if j.kind == "rotq4"]
        given = [j for j in jobs if j.kind == "q4"]
        for group, fused in ((rot, True), (given, False)):
            if not group:
                continue
            shapes = [tuple(j.state["weight"].shape) for j in group]
            words = _Arena(sum(_up(r * c // 2) for r, c in shapes), dev)
            packed = [words.take((r, c // 8), torch.int32) for r, c in shapes]
            if fused:
                sarena = _Arena(sum(_up(r * c // 64) for r, c in shapes), dev)
                scales = [sarena.take((r, c // 128), torch.bfloat16) for r, c in shapes]
            else:
                scales = [j.state["weight_scale"].contiguous() for j in group]
            ins = [j.state["weight"].contiguous() for j in group]
            table = _table(ins, packed, scales, shapes)
            stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
            if fused:
                # groups of jobs that share one sign vector (one transform weight per size: normally a single group)
                by_signs: Dict[int, List[int]] = {}
                for i, j in enumerate(group):
                    by_signs.setdefault(id(j.transforms[0].weight), []).append(i)
                for idxs in by_signs.values():
                    signs = self._signs_on(group[idxs[0]].transforms[0], dev)
                    sub = np.ascontiguousarray(table[idxs])
                    with self._timed("compress", dev):
                        L.check(L.lib().ctb_rotate_quantize_int4_batch(_table_ptr(sub), L.i32(len(idxs)), L.ptr(signs),
                                                                       L.i32(ops._precision_code(self.rotation_precision)),
                                                                       L.ptr(self._status_word(dev)), stream))
                    self.launches += 1
            else:
                with self._timed("compress", dev):
                    L.check(L.lib().ctb_quantize_pack_int4_batch(_table_ptr(table), L.i32(len(group)), stream))
                self.launches += 1
            shape_rows = torch.tensor(shapes).unbind(0)  # int64 [2] each, as torch.tensor(weight.shape)
            for j, p, s, shp, srow in zip(group, packed, scales, shapes, shape_rows):
                j.out = {"weight_shape": srow, "weight_packed": p}
                if fused:
                    j.qparams = {"weight_scale": s}
                j.shape, j.quantized = shp, True
        group = [j for j in jobs if j.kind == "q8c"]
        if group:
            shapes = [tuple(j.state["weight"].shape) for j in group]
            codes = _Arena(sum(_up(r * c) for r, c in shapes), dev)
            outs = [codes.take((r, c), torch.float8_e4m3fn) for r, c in shapes]
            table = _table([j.state["weight"].contiguous() for j in group], outs,
                           [j.state["weight_scale"].contiguous() for j in group], shapes)
            zps = [j.state.get("weight_zero_point") for j in group]
            zps = [None if z is None else z.contiguous() for z in zps]
            with self._timed("compress", dev):
                self._fp8_quantize(table, zps, dev)
            self.launches += 1
            for j, o, shp in zip(group, outs, shapes):
                j.out = {"weight": o}
                j.shape, j.quantized = shp, True
        group = [j for j in jobs if j.kind == "q4f"]
        if group:
            shapes = [tuple(j.state["weight"].shape) for j in group]
            codes = _Arena(sum(_up(r * c // 2) for r, c in shapes), dev)
            outs = [codes.take((r, c // 2), torch.uint8) for r, c in shapes]
            table = _table([j.state["weight"].contiguous() for j in group], outs,
                           [j.state["weight_scale"].contiguous() for j in group], shapes)
            gss = [j.state["weight_global_scale"].contiguous() for j in group]
            zps = [j.state.get("weight_zero_point") for j in group]
            zps = [None if z is None else z.contiguous() for z in zps]
            with self._timed("compress", dev):
                ops.quantize_fp4_g16_batch(_table_ptr(table), gss, zps, device=dev)
            self.launches += 1
            for j, o, shp in zip(group, outs, shapes):
                j.out = {"weight_packed": o}
                j.shape, j.quantized = shp, True
        for j in jobs:
            if j.kind == "generic":
                self._compress_generic(j)

    def _fp8_quantize(self, table: np.ndarray, zps, dev: torch.device) -> None:
        stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
        arr, zdt = None, 0
        if any(z is not None for z in zps):
            dts = {z.dtype for z in zps if z is not None}
            if len(dts) != 1:
                raise TypeError("zero points of one shard must share one dtype")
            zdt = L.DT[next(iter(dts))]
            arr = (ctypes.c_void_p * len(zps))(*[None if z is None else z.data_ptr() for z in zps])
        L.check(L.lib().ctb_quantize_fp8_channel_batch(_table_ptr(table), L.i32(len(table)), arr, L.i32(zdt), stream))

    def _compress_generic(self, j: Job) -> None:
        """The per-tensor walk on device tensors: fuse pending transforms, calibrate where a rotation invalidated
        the scales, then the registered compressor (quantized_compressors/base.py:91-134)."""
        st = dict(j.state)
        w = st.get("weight")
        if w is not None and j.transforms:
            for tr in j.transforms:
                w = tr(w)
            st["weight"] = w
            if j.scheme is not None and j.scheme.weights is not None:
                st.update(minmax_qparams(w, j.scheme.weights))
        if w is not None and j.transforms:
            j.qparams = {k: st[k] for k in _QPARAMS if k in st and st[k] is not j.state.get(k)}
        if w is not None and self._fp8_sparse24(j, w, st):
            return
        if w is not None and j.compressor is not None and j.scheme is not None and j.scheme.weights is not None \
                and st.get("weight_scale") is not None:
            j.out = dict(j.compressor.compress_weight(weight=w, scale=st["weight_scale"], zero_point=st.get("weight_zero_point"),
                                                      global_scale=st.get("weight_global_scale"), g_idx=st.get("weight_g_idx"),
                                                      quantization_args=j.scheme.weights, device=None))
            j.shape, j.quantized = tuple(w.shape), True
        elif w is not None and j.transforms:
            j.out = {"weight": w}

    def _fp8_sparse24(self, j: Job, w: Tensor, st: Dict[str, Tensor]) -> bool:
        """A weight that the float-quantized compressor would turn into per-channel FP8 and the sparse-24-bitmask
        compressor would then compact (model_compressor.py:498-519) goes through one kernel; the FP8 tensor between
        the two is never materialised.  Fills the job as the two compressors would have."""
        args = j.scheme.weights if j.scheme is not None else None
        scale = st.get("weight_scale")
        if (not self.fuse_sparse24 or not j.sparse or j.compressor is None or args is None or scale is None
                or getattr(j.compressor, "_format_name", None) != CompressionFormat.float_quantized.value
                or args.type != QuantizationType.FLOAT or args.num_bits != 8 or args.strategy != QuantizationStrategy.CHANNEL
                or args.dynamic or w.ndim != 2 or w.dtype != torch.bfloat16 or not w.is_cuda or w.shape[1] % 8
                or scale.dtype != torch.bfloat16 or scale.numel() != w.shape[0]
                or st.get("weight_g_idx") is not None or st.get("weight_global_scale") is not None):
            return False
        zp = st.get("weight_zero_point")
        if zp is not None and (zp.numel() != w.shape[0] or zp.dtype not in L.DT):
            return False
        with self._timed("compress", w.device):
            values, bitmask = ops.quantize_fp8_sparse24(w, scale, zp)
        self.launches += 1
        j.out, j.shape, j.quantized = {}, tuple(w.shape), True
        j.sparse_out = {"shape": torch.tensor(list(w.shape)).reshape(-1, 1), "compressed": values, "bitmask": bitmask}
        return True

    # ------------------------------------------------------------------ decompress
    def classify_decompress(self, job: Job) -> None:
        job.kind = "generic"
        if job.compressor is None or job.scheme is None or job.sparse:
            return
        fmt = getattr(job.compressor, "_format_name", None)
        q = job.state.get("weight")
        if (q is not None and q.ndim == 2 and q.dtype == torch.float8_e4m3fn and job.state.get("weight_zero_point") is None
                and self._is_fp8_channel(job, fmt, job.scheme.weights, q.shape[0], q.shape[1])):
            job.kind, job.shape = "dq8c", tuple(q.shape)
            return
        p, s = job.state.get("weight_packed"), job.state.get("weight_scale")
        if (p is not None and p.ndim == 2 and p.dtype == torch.uint8 and job.state.get("weight_zero_point") is None
                and self._is_nvfp4(job, fmt, job.scheme.weights, p.shape[0], 2 * p.shape[1])):
            job.kind, job.shape = "dq4f", (p.shape[0], 2 * p.shape[1])
            return
        if (fmt != CompressionFormat.pack_quantized.value or not is_w4a16_g128(job.scheme.weights) or p is None or s is None
                or p.dtype != torch.int32 or s.dtype != torch.bfloat16 or p.ndim != 2 or s.ndim != 2):
            return
        if job.state.get("weight_g_idx") is not None or job.state.get("weight_zero_point") is not None:
            return
        rows, cols = p.shape[0], s.shape[1] * 128
        if p.shape[1] * 8 != cols or s.shape[0] != rows:
            return
        job.kind, job.shape = "dq4", (rows, cols)

    def _decompress_on_device(self, jobs: List[Job], dev: torch.device, sparsity_compressor=None) -> None:
        group = [j for j in jobs if j.kind == "dq4"]
        if group:
            shapes = [j.shape for j in group]
            dense = _Arena(sum(_up(r * c * 2) for r, c in shapes), dev)
            outs = [dense.take((r, c), torch.bfloat16) for r, c in shapes]
            table = _table([j.state["weight_packed"].contiguous() for j in group], outs,
                           [j.state["weight_scale"].contiguous() for j in group], shapes)
            stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
            with self._timed("decompress", dev):
                L.check(L.lib().ctb_unpack_dequantize_int4_batch(_table_ptr(table), L.i32(len(group)), stream))
            self.launches += 1
            for j, o in zip(group, outs):
                j.out = {"weight": o}
        group = [j for j in jobs if j.kind == "dq8c"]
        if group:
            shapes = [j.shape for j in group]
            dense = _Arena(sum(_up(r * c * 2) for r, c in shapes), dev)
            outs = [dense.take((r, c), torch.bfloat16) for r, c in shapes]
            table = _table([j.state["weight"].contiguous() for j in group], outs,
                           [j.state["weight_scale"].contiguous() for j in group], shapes)
            stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
            with self._timed("decompress", dev):
                L.check(L.lib().ctb_dequantize_fp8_channel_batch(_table_ptr(table), L.i32(len(group)), stream))
            self.launches += 1
            for j, o in zip(group, outs):
                j.out = {"weight": o}
        group = [j for j in jobs if j.kind == "dq4f"]
        if group:
            shapes = [j.shape for j in group]
            dense = _Arena(sum(_up(r * c * 2) for r, c in shapes), dev)
            outs = [dense.take((r, c), torch.bfloat16) for r, c in shapes]
            table = _table([j.state["weight_packed"].contiguous() for j in group], outs,
                           [j.state["weight_scale"].contiguous() for j in group], shapes)
            gss = [j.state["weight_global_scale"].contiguous() for j in group]
            with self._timed("decompress", dev):
                ops.dequantize_fp4_g16_batch(_table_ptr(table), gss, device=dev)
            self.launches += 1
            for j, o in zip(group, outs):
                j.out = {"weight": o}
        for j in jobs:
            if j.kind != "generic":
                continue
            st = dict(j.state)
            if j.sparse and sparsity_compressor is not None and self._sparse24_fp8(j, st):
                continue
            if j.sparse and sparsity_compressor is not None:
                names = sparsity_compressor.compression_param_names
                data = {k: v for k, v in st.items() if k in names}
                if data:
                    st = {k: v for k, v in st.items() if k not in names}
                    st["weight"] = sparsity_compressor.decompress_weight(data)
            out = {}
            if j.compressor is not None and j.scheme is not None and "weight_scale" in st and j.scheme.weights is not None:
                out["weight"] = j.compressor.decompress_weight(compressed_data=st, quantization_args=j.scheme.weights)
            elif "weight" in st and st["weight"] is not j.state.get("weight"):
                out["weight"] = st["weight"]
            j.out = out

    def _sparse24_fp8(self, j: Job, st: Dict[str, Tensor]) -> bool:
        """The inverse of _fp8_sparse24: kept e4m3 values + bitmask of a sparse-24-bitmask module whose scheme is FP8
        per channel go to the bf16 weight in one kernel (model_compressor.py:580-611 does it in two walks)."""
        args = j.scheme.weights if j.scheme is not None else None
        vals, bm, shape, scale = st.get("compressed"), st.get("bitmask"), st.get("shape"), st.get("weight_scale")
        if (not self.fuse_sparse24 or j.compressor is None or args is None or vals is None or bm is None or shape is None or scale is None
                or getattr(j.compressor, "_format_name", None) != CompressionFormat.float_quantized.value
                or args.type != QuantizationType.FLOAT or args.num_bits != 8 or args.strategy != QuantizationStrategy.CHANNEL
                or args.dynamic or vals.dtype != torch.float8_e4m3fn or not vals.is_cuda or scale.dtype != torch.bfloat16
                or st.get("weight_zero_point") is not None or st.get("weight_g_idx") is not None):
            return False
        rows, cols = (int(v) for v in shape.flatten().tolist())  # a small host tensor (the reference stores the shape as one)
        if cols % 8 or scale.numel() != rows or tuple(bm.shape) != (rows, cols // 8):
            return False
        with self._timed("decompress", vals.device):
            w = ops.sparse24_decompress_dequantize_fp8(vals, bm, scale, (rows, cols))
        self.launches += 1
        j.out = {"weight": w}
        return True

    # ------------------------------------------------------------------ replay of a recorded cycle
    def replay_compress(self, table: np.ndarray, signs: Tensor, dev: torch.device) -> None:
        """The fused rotate + calibrate + quantize + pack launch over a table recorded by an earlier pass."""
        self._check_status(wait=False)
        stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
        with self._timed("compress", dev):
            L.check(L.lib().ctb_rotate_quantize_int4_batch(_table_ptr(table), L.i32(len(table)), L.ptr(signs),
                                                           L.i32(ops._precision_code(self.rotation_precision)),
                                                           L.ptr(self._status_word(dev)), stream))
        self.launches += 1

    def replay_decompress(self, table: np.ndarray, dev: torch.device) -> None:
        stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
        with self._timed("decompress", dev):
            L.check(L.lib().ctb_unpack_dequantize_int4_batch(_table_ptr(table), L.i32(len(table)), stream))
        self.launches += 1

    # ------------------------------------------------------------------ drivers
    def run(self, jobs: List[Job], direction: str, deliver: Optional[str] = None, sparsity_compressor=None,
            sparse_compress: Optional[Callable[[Job], None]] = None) -> None:
        """Process `jobs` ("compress" or "decompress").  Results (job.out) are left on the device of the job's
        weight, or in page-locked host memory for host-resident jobs and when `deliver` is "cpu"."""
        work = self._compress_on_device if direction == "compress" else (
            lambda js, d: self._decompress_on_device(js, d, sparsity_compressor))
        self._check_status(wait=False)  # a time-out reported by an earlier, purely device-side call surfaces here
        host_side = False
        by_dev: Dict[Optional[int], List[Job]] = {}
        for j in jobs:
            t = _anchor(j)
            by_dev.setdefault(t.device.index if (t is not None and t.is_cuda) else None, []).append(j)
        for idx, js in by_dev.items():
            if idx is None:
                self._run_host(js, work, direction, sparse_compress)
                host_side = True
            else:
                dev = torch.device("cuda", idx)
                with torch.cuda.device(dev):
                    work(js, dev)
                    if sparse_compress is not None:
                        for j in js:
                            sparse_compress(j)
                    if deliver == "cpu":
                        self._deliver_host(js, dev)
                        host_side = True
        # Device-resident work is ordered on the caller's stream like any torch op and needs no host wait; results
        # that land in host memory are waited for here unless the caller deferred that (`deferred`).
        if host_side and not self.deferred:
            self.finish()

    def _deliver_host(self, jobs: List[Job], dev: torch.device) -> None:
        cur = torch.cuda.current_stream(dev)
        total = sum(_up(_nbytes(v)) for j in jobs for _, _, v in j.results() if v.is_cuda)
        host = _Arena(total, pinned=True)
        for j in jobs:
            for d, k, v in j.results():
                if v.is_cuda:
                    h = host.take(v.shape, v.dtype)
                    h.copy_(v.contiguous(), non_blocking=True)
                    d[k] = h
        ev = torch.cuda.Event()
        ev.record(cur)
        self._tail.append(ev)

    def _run_host(self, jobs: List[Job], work, direction: str, sparse_compress) -> None:
        """Host-resident jobs: steps of about STEP_BYTES streamed over three streams of the current device.

        A step whose outputs are known without running it (every job goes through a whole-shard entry point) is
        *planned*: its page-locked output tensors exist at once, so the caller can hang them on the model, while its
        copies and launches are *submitted* either right away or, when the caller deferred synchronisation, in an
        order that interleaves the passes it has requested so far (`_drain`).  The order matters: copies of one
        direction run in the order they were submitted, whatever stream they are on, so a decompress pass queued
        wholesale behind a compress pass would see its small uploads wait behind every weight of the model."""
        if not torch.cuda.is_available():
            raise RuntimeError("compressed_tensors_b200 needs a CUDA device (no CPU fallback)")
        dev = torch.device("cuda", torch.cuda.current_device())

        # steps by the larger side of the job (what comes in when compressing, what goes out when decompressing), so
        # that a step is a few hundred megabytes on the bus in its long direction whatever the compression ratio
        def weight_of(j: Job) -> int:
            nin = sum(_nbytes(v) for v in self._inputs_of(j, direction).values())
            if direction == "compress":
                return nin
            if j.shape is not None:
                return max(nin, 2 * j.shape[0] * j.shape[1])
            return 4 * nin

        groups: List[List[Job]] = [[]]
        acc = 0
        for j in jobs:
            nb = weight_of(j)
            if groups[-1] and acc + nb > STEP_BYTES:
                groups.append([])
                acc = 0
            groups[-1].append(j)
            acc += nb
        for group in groups:
            if not group:
                continue
            step = _Step(direction, group, dev, work, sparse_compress, need=2 * sum(weight_of(j) for j in group))
            step.feeds = [self._inputs_of(j, direction) for j in group]
            step.reads = {h.untyped_storage().data_ptr() for f in step.feeds for h in f.values()}
            if all(j.kind in _PLANNED_KINDS for j in group) and sparse_compress is None:
                self._plan(step)
                self._queue.append(step)
                # Deferred: hold the step back so that a pass requested later can be interleaved with this one; the
                # first two steps of a lone pass would lead any interleaving, so they go out at once and the GPU starts.
                lone = all(q.direction == direction for q in self._queue)
                if not self.deferred or (lone and sum(1 for q in self._queue) <= 2 and self._eager_head.get(direction, 0) < 2):
                    if self.deferred:
                        self._eager_head[direction] = self._eager_head.get(direction, 0) + 1
                    self._drain()
            else:
                self._drain()  # whatever was planned before comes first
                self._submit(step)

    def _plan(self, step: "_Step") -> None:
        """Create the host-side results of a step (views of one page-locked block) without running it."""
        specs = []  # (job, dict, name, shape, dtype)
        for j in step.jobs:
            if step.direction == "compress" and j.kind == "q8c":
                r, c = j.state["weight"].shape
                j.out = {}
                specs.append((j, j.out, "weight", (r, c), torch.float8_e4m3fn))
                j.shape, j.quantized = (r, c), True
            elif step.direction == "compress" and j.kind == "q4f":
                r, c = j.state["weight"].shape
                j.out = {}
                specs.append((j, j.out, "weight_packed", (r, c // 2), torch.uint8))
                j.shape, j.quantized = (r, c), True
            elif step.direction == "compress":
                r, c = j.state["weight"].shape
                j.out = {"weight_shape": torch.tensor((r, c))}  # int64 [2], as torch.tensor(weight.shape)
                specs.append((j, j.out, "weight_packed", (r, c // 8), torch.int32))
                if j.kind == "rotq4":
                    specs.append((j, j.qparams, "weight_scale", (r, c // 128), torch.bfloat16))
                j.shape, j.quantized = (r, c), True
            else:
                specs.append((j, j.out, "weight", j.shape, torch.bfloat16))
        host = _Arena(sum(_up(_prod(shape) * _ITEMSIZE[dt]) for _, _, _, shape, dt in specs), pinned=True)
        for j, d, name, shape, dt in specs:
            d[name] = host.take(shape, dt)
            step.planned.append((j, d is j.qparams, name, d[name]))
        step.writes = host.buf.untyped_storage().data_ptr()
        self._producer[step.writes] = step

    def _drain(self) -> None:
        """Submit the planned steps.  Passes are interleaved: a step is submitted as soon as every step that produces
        what it reads has been submitted and, so that the copy engine never has to wait for that round trip, one more
        step of the producing pass behind them; steps of one pass keep their order."""
        queue, self._queue = self._queue, []
        passes: Dict[str, List[_Step]] = {}
        for st in queue:
            passes.setdefault(st.direction, []).append(st)
        order = list(passes)  # the order in which the passes were requested
        while any(passes.values()):
            progressed = False
            for d in reversed(order):  # the later pass first: its steps are the ones that wait on others
                if not passes[d]:
                    continue
                st = passes[d][0]
                producers = [self._producer[p] for p in st.reads if p in self._producer]
                pending = [q for q in producers if not q.submitted]
                if pending:
                    continue
                # keep the producing pass one step ahead
                ahead_ok = True
                for q in producers:
                    rest = passes.get(q.direction, [])
                    if rest and d != q.direction and not self._lead_ok(q, rest):
                        ahead_ok = False
                if not ahead_ok:
                    continue
                self._submit(passes[d].pop(0))
                progressed = True
                break
            if not progressed:
                # nothing of a later pass is ready: advance the earliest pass that has steps left
                for d in order:
                    if passes[d]:
                        self._submit(passes[d].pop(0))
                        break

    @staticmethod
    def _lead_ok(producer: "_Step", rest: List["_Step"]) -> bool:
        """True when the pass of `producer` has submitted at least one step after it (or has none left)."""
        return producer.successor_submitted or not rest

    def _submit(self, step: "_Step") -> None:
        dev, direction = step.dev, step.direction
        s_in, s_k, s_out = self._get_streams(dev, direction)
        # The host only enqueues; it waits for an old step when the device buffers of the steps still in flight would
        # outgrow the budget (inputs plus outputs: outputs are at most the inputs when compressing, a few times when not).
        if self._budget.get(dev.index) is None:
            self._budget[dev.index] = INFLIGHT_FRACTION * torch.cuda.mem_get_info(dev)[0]
        inflight = self._inflight.setdefault(dev.index, [])
        while inflight and sum(nb for _, nb in inflight) + step.need > self._budget[dev.index]:
            ev, _ = inflight.pop(0)
            ev.synchronize()
        ev_in, ev_k, ev_out = torch.cuda.Event(), torch.cuda.Event(), torch.cuda.Event()
        originals = []
        planned_out = [(j, j.out, j.qparams) for j in step.jobs] if step.planned else None
        with torch.cuda.device(dev):
            with torch.cuda.stream(s_in):
                arena = _Arena(sum(_up(_nbytes(v)) for f in step.feeds for v in f.values()), dev)
                for j, f in zip(step.jobs, step.feeds):
                    originals.append(j.state)
                    st = dict(j.state)
                    for name, h in f.items():
                        ready = self._host_ready.get(h.untyped_storage().data_ptr())
                        if ready is not None:
                            s_in.wait_event(ready)  # bytes an earlier step is still delivering
                        d = arena.take(h.shape, h.dtype)
                        d.copy_(h, non_blocking=True)
                        st[name] = d
                    j.state = st
                ev_in.record(s_in)
            arena.buf.record_stream(s_k)
            with torch.cuda.stream(s_k):
                s_k.wait_event(ev_in)
                if step.planned:
                    for j in step.jobs:
                        j.out, j.qparams = {}, {}
                step.work(step.jobs, dev)
                if step.sparse_compress is not None:
                    for j in step.jobs:
                        step.sparse_compress(j)
                ev_k.record(s_k)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_k)
                if step.planned:
                    for j, in_qparams, name, h in step.planned:
                        v = (j.qparams if in_qparams else j.out)[name]
                        if tuple(v.shape) != tuple(h.shape) or v.dtype != h.dtype:
                            raise RuntimeError(f"{j.prefix}.{name}: planned {tuple(h.shape)} {h.dtype}, produced {tuple(v.shape)} {v.dtype}")
                        v = v.contiguous()
                        v.record_stream(s_out)
                        h.copy_(v, non_blocking=True)
                    for (j, out, qparams) in planned_out:
                        j.out, j.qparams = out, qparams  # the host tensors the caller already holds
                    ev_out.record(s_out)
                    self._host_ready[step.writes] = ev_out
                else:
                    outs = [(d, name, v) for j in step.jobs for d, name, v in j.results() if v.is_cuda]  # small host tensors (shapes) stay
                    host = _Arena(sum(_up(_nbytes(v)) for _, _, v in outs), pinned=True)
                    for d, name, v in outs:
                        v = v.contiguous()
                        v.record_stream(s_out)
                        h = host.take(v.shape, v.dtype)
                        h.copy_(v, non_blocking=True)
                        d[name] = h
                    ev_out.record(s_out)
                    if outs:
                        self._host_ready[host.buf.untyped_storage().data_ptr()] = ev_out
        for j, orig in zip(step.jobs, originals):
            j.state = orig
        step.submitted = True
        if step.direction in self._last_submitted:
            self._last_submitted[step.direction].successor_submitted = True
        self._last_submitted[step.direction] = step
        inflight.append((ev_out, step.need))
        self._tail.append(ev_out)

    @staticmethod
    def _inputs_of(j: Job, direction: str) -> Dict[str, Tensor]:
        """The host tensors a job needs on the device."""
        if direction == "compress":
            names = ("weight",) + _QPARAMS
        else:
            names = ("weight_packed", "weight_scale", "weight_zero_point", "weight_g_idx", "weight_global_scale", "weight_shape",
                     "weight", "compressed", "bitmask", "row_offsets", "shape", "meta", "scale_packed")
        out = {}
        for n in names:
            t = j.state.get(n)
            if t is not None and not t.is_cuda and t.device.type == "cpu":
                if direction == "decompress" and n in ("weight_shape", "shape"):
                    continue  # read on the host
                out[n] = t
        return out


def _anchor(j: Job) -> Optional[Tensor]:
    for n in ("weight", "weight_packed", "compressed", "bitmask"):
        t = j.state.get(n)
        if t is not None:
            return t
    for t in j.state.values():
        return t
    return None


def _fusable_rotation(tr) -> bool:
    """A block-128, forward, unpermuted weight_input Hadamard rotation of a Linear weight: what the fused
    rotate + calibrate + quantize + pack kernels implement."""
    from ...transform.transform_args import TransformLocation

    try:
        return (TransformLocation(tr.args.location) == TransformLocation.WEIGHT_INPUT and not tr.args.inverse
                and tr.perm is None and tr.module_type == torch.nn.Linear and tr.weight.size(0) == 128)
    except AttributeError:
        return False
