"""Partitioning of a whole-model compress / decompress over the GPUs of one node.

The reference walks the state dict one tensor at a time on one CPU
(compressors/quantized_compressors/base.py:69-134, model_compressors/model_compressor.py:453-617).
Every weight is an independent unit of work, so the walk shards with no data-path collective:
decoder layers are dealt to ranks in contiguous blocks and each rank runs the fused kernels on its
own tensors.  A collective is needed only when ONE tensor's reduction is split across ranks (the
NVFP4 global scale / TENSOR strategy); `allreduce_amax` covers that case with a 4-byte
all-reduce(max), which is exact and order independent, so results do not depend on the world size.
"""
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch

__all__ = ["LLAMA3_8B", "ModelShape", "linear_shapes", "partition_layers", "allreduce_amax", "ShardCodec", "HostRoundTrip"]


@dataclass(frozen=True)
class ModelShape:
    layers: int
    hidden: int
    intermediate: int
    q_heads: int
    kv_heads: int
    head_dim: int
    vocab: int


LLAMA3_8B = ModelShape(layers=32, hidden=4096, intermediate=14336, q_heads=32, kv_heads=8, head_dim=128, vocab=128256)


def linear_shapes(m: ModelShape) -> List[Tuple[str, int, int]]:
    """(name, out_features, in_features) of the Linear weights of one decoder layer."""
    kv = m.kv_heads * m.head_dim
    q = m.q_heads * m.head_dim
    return [
        ("self_attn.q_proj", q, m.hidden),
        ("self_attn.k_proj", kv, m.hidden),
        ("self_attn.v_proj", kv, m.hidden),
        ("self_attn.o_proj", m.hidden, q),
        ("mlp.gate_proj", m.intermediate, m.hidden),
        ("mlp.up_proj", m.intermediate, m.hidden),
        ("mlp.down_proj", m.hidden, m.intermediate),
    ]


def partition_layers(num_layers: int, world_size: int, rank: int) -> range:
    """Contiguous block of layers owned by `rank`; the first `num_layers % world_size` ranks get one more."""
    if world_size <= 0 or not (0 <= rank < world_size):
        raise ValueError(f"bad rank {rank} for world size {world_size}")
    base, extra = divmod(num_layers, world_size)
    start = rank * base + min(rank, extra)
    return range(start, start + base + (1 if rank < extra else 0))


def allreduce_amax(min_val: torch.Tensor, max_val: torch.Tensor, group=None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Combine per-rank (min, max) of a tensor that is split across ranks.  No-op without a process group."""
    import torch.distributed as dist

    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return min_val, max_val
    # one message: [max, -min] reduced with MAX (fp32 holds bf16/fp16/fp32 extrema exactly)
    buf = torch.stack([max_val.float().reshape(()), -min_val.float().reshape(())])
    dist.all_reduce(buf, op=dist.ReduceOp.MAX, group=group)
    return (-buf[1]).to(min_val.dtype).reshape(min_val.shape), buf[0].to(max_val.dtype).reshape(max_val.shape)


class ShardCodec:
    """Pre-planned compress / decompress of one rank's weights: random-Hadamard rotation (block
    `hadamard_n`, weight_input) fused with W4A16 group quantize + pack_to_int32, and the inverse
    unpack + dequantize.  Output buffers are allocated once; `use_graphs` replays the launches from
    CUDA graphs so that a shard of many small tensors is not bound by launch latency."""

    def __init__(self, weights: Sequence[torch.Tensor], *, group_size: int = 128, hadamard_n: int = 128,
                 signs: Optional[torch.Tensor] = None, precision=torch.float64, use_graphs: bool = False, batch: bool = True):
        from . import ops

        self.ops = ops
        self.weights = list(weights)
        self.group_size, self.hadamard_n, self.precision = group_size, hadamard_n, precision
        dev = self.weights[0].device
        self.signs = None if signs is None else signs.to(device=dev, dtype=torch.int8)
        self.packed: List[Optional[torch.Tensor]] = [None] * len(self.weights)
        self.scales: List[Optional[torch.Tensor]] = [None] * len(self.weights)
        self.restored: List[Optional[torch.Tensor]] = [None] * len(self.weights)
        self._graphs: Dict[str, torch.cuda.CUDAGraph] = {}
        self.use_graphs = use_graphs
        self.batch = batch
        # set to CTB_ETIMEOUT by the tensor-core kernel if one of its bounded waits gives up
        self.status = torch.zeros(1, dtype=torch.int32, device=dev)

    # ------------------------------------------------------------------ launches
    def _allocate(self) -> None:
        if self.packed[0] is not None:
            return
        dev = self.weights[0].device
        for i, w in enumerate(self.weights):
            rows, cols = w.shape
            self.packed[i] = torch.empty((rows, cols // 8), dtype=torch.int32, device=dev)
            self.scales[i] = torch.empty((rows, cols // self.group_size), dtype=w.dtype, device=dev)
            self.restored[i] = torch.empty_like(w)
        shapes = [tuple(w.shape) for w in self.weights]
        self._ctable = self.ops.tensor_table(self.weights, self.packed, self.scales, shapes)
        self._dtable = self.ops.tensor_table(self.packed, self.restored, self.scales, shapes)

    @property
    def batched(self) -> bool:
        """One grid for the whole shard (block-128 rotation, group 128, bf16); otherwise one launch per tensor."""
        return (self.batch and self.hadamard_n == 128 and self.group_size == 128
                and all(w.dtype == torch.bfloat16 and w.shape[1] % 128 == 0 for w in self.weights))

    def _compress(self) -> None:
        if self.batched:
            self._allocate()
            self.ops.rotate_quantize_int4_batch(self._ctable, self.signs, self.precision, self.weights[0].device, self.status)
            return
        for i, w in enumerate(self.weights):
            self.packed[i], self.scales[i] = self.ops.absmax_quantize(
                w, qtype=self.ops.QINT, bits=4, col_group=self.group_size, codec="pack32",
                hadamard_n=self.hadamard_n, signs=self.signs, precision=self.precision)

    def _decompress(self) -> None:
        if self.batched:
            self._allocate()
            self.ops.unpack_dequantize_int4_batch(self._dtable, self.weights[0].device)
            return
        for i, w in enumerate(self.weights):
            cols = w.shape[1]
            self.restored[i] = self.ops.dequantize(
                self.packed[i], self.scales[i], None, qtype=self.ops.QINT, bits=4, col_group=self.group_size,
                scale_row_stride=cols // self.group_size, out_dtype=w.dtype, codec="pack32", cols=cols)

    # ------------------------------------------------------------------ graph replay
    def _run(self, name: str, fn) -> None:
        if not self.use_graphs:
            fn()
            return
        g = self._graphs.get(name)
        if g is None:
            fn()  # warm-up outside capture (first call may initialise library state)
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                fn()
            self._graphs[name] = g
        g.replay()

    def compress(self) -> None:
        self._run("compress", self._compress)

    def decompress(self) -> None:
        self._run("decompress", self._decompress)

    # ------------------------------------------------------------------ accounting
    @property
    def numel(self) -> int:
        return sum(w.numel() for w in self.weights)

    @property
    def launches_per_pass(self) -> int:
        return -(-len(self.weights) // 256) if self.batched else len(self.weights)


class HostRoundTrip:
    """End-to-end compress + decompress of a shard whose tensors live in (pinned) HOST memory, the way the
    reference's ModelCompressor sees a CPU state dict: weights go host -> device, packed words and scales come
    back to the host, and the decompress half reads those host buffers again and returns dense weights to the
    host.  Work is cut into groups of tensors (one decoder layer each) and spread over three streams -- copy-in,
    kernels, copy-out -- so that both PCIe directions and the GPU stay busy at once; events carry the
    dependencies (a group is decompressed only after its own packed bytes made the trip to the host and back)."""

    def __init__(self, host_weights: Sequence[torch.Tensor], group: int, device, *, signs=None, precision=torch.float64, ramp: int = 0):
        """`group` tensors per pipeline step; the first and last `ramp` tensors go one per step, which shortens the
        stretch at either end of the trip during which only one copy direction has work."""
        self.device = torch.device(device)
        self.host_w = list(host_weights)
        n = len(self.host_w)
        ramp = max(0, min(ramp, n // 2))
        self.groups = [[i] for i in range(ramp)]
        self.groups += [list(range(i, min(i + group, n - ramp))) for i in range(ramp, n - ramp, group)]
        self.groups += [[i] for i in range(n - ramp, n)]
        self.dev_w = [torch.empty(w.shape, dtype=w.dtype, device=self.device) for w in self.host_w]
        self.codecs = [ShardCodec([self.dev_w[i] for i in g], signs=signs, precision=precision) for g in self.groups]
        for c in self.codecs:
            if not c.batched:
                raise NotImplementedError("the host round trip is built for the batched bf16 / block-128 / group-128 path")
            c._allocate()
        pin = dict(pin_memory=True)
        self.host_p = [torch.empty((w.shape[0], w.shape[1] // 8), dtype=torch.int32, **pin) for w in self.host_w]
        self.host_s = [torch.empty((w.shape[0], w.shape[1] // 128), dtype=w.dtype, **pin) for w in self.host_w]
        self.host_r = [torch.empty(w.shape, dtype=w.dtype, **pin) for w in self.host_w]
        self.s_in, self.s_k, self.s_out = (torch.cuda.Stream(self.device) for _ in range(3))

    @property
    def h2d_bytes(self) -> int:
        return sum(w.numel() * w.element_size() for w in self.host_w) + self.d2h_packed_bytes

    @property
    def d2h_packed_bytes(self) -> int:
        return sum(p.numel() * 4 for p in self.host_p) + sum(s.numel() * s.element_size() for s in self.host_s)

    @property
    def d2h_bytes(self) -> int:
        return self.d2h_packed_bytes + sum(w.numel() * w.element_size() for w in self.host_w)

    def run(self) -> None:
        """One round trip of the whole shard; returns after everything has landed in the host buffers.

        Two stages per group, issued one group apart so that neither copy direction ever waits on the other:
          A(k): weights host -> device, compress, packed bytes device -> host;
          B(k): packed bytes host -> device, decompress, dense weights device -> host.
        Issue order A(0), A(1), B(0), A(2), B(1), ...: the copy-in stream then carries W0 W1 P0 W2 P1 ... and the
        copy-out stream P0 P1 R0 P2 R1 ..., i.e. the small packed transfer of the NEXT group is already through
        when the large dense transfer of this group starts, and the packed bytes a B stage needs back are on the
        host long before its turn."""
        ev = torch.cuda.Event
        n = len(self.groups)
        packed_on_host = [None] * n

        def stage_a(k):
            g, codec = self.groups[k], self.codecs[k]
            e_in, e_c, e_o = ev(), ev(), ev()
            with torch.cuda.stream(self.s_in):
                for i in g:
                    self.dev_w[i].copy_(self.host_w[i], non_blocking=True)
                e_in.record()
            with torch.cuda.stream(self.s_k):
                self.s_k.wait_event(e_in)
                codec._compress()
                e_c.record()
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(e_c)
                for j, i in enumerate(g):
                    self.host_p[i].copy_(codec.packed[j], non_blocking=True)
                    self.host_s[i].copy_(codec.scales[j], non_blocking=True)
                e_o.record()
            packed_on_host[k] = e_o

        def stage_b(k):
            g, codec = self.groups[k], self.codecs[k]
            e_in2, e_d = ev(), ev()
            with torch.cuda.stream(self.s_in):
                self.s_in.wait_event(packed_on_host[k])  # the packed bytes made it to the host: bring them back
                for j, i in enumerate(g):
                    codec.packed[j].copy_(self.host_p[i], non_blocking=True)
                    codec.scales[j].copy_(self.host_s[i], non_blocking=True)
                e_in2.record()
            with torch.cuda.stream(self.s_k):
                self.s_k.wait_event(e_in2)
                codec._decompress()
                e_d.record()
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(e_d)
                for j, i in enumerate(g):
                    self.host_r[i].copy_(codec.restored[j], non_blocking=True)

        for k in range(n + 1):
            if k < n:
                stage_a(k)
            if k >= 1:
                stage_b(k - 1)
        for s in (self.s_in, self.s_k, self.s_out):
            s.synchronize()
