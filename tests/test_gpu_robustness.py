"""Error paths and bounds, exercised without faulting the GPU: a device-side wait that is made to run out returns
a status and leaves the context usable; a value buffer shorter than the fast 2:4 kernels assume is routed to the
kernels that read exactly what the bitmask has; one process driving two devices."""
import ctypes

import pytest
import torch

from tests.helpers import assert_bit_equal

pytestmark = pytest.mark.gpu


def weights(rows, cols, seed, std=0.02):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(rows, cols, generator=g) * std).to(torch.bfloat16)


def signs128(seed=0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randint(0, 2, (128,), generator=g) * 2 - 1).to(torch.int8)


def test_tensor_core_kernel_wait_runs_out_and_returns():
    """The tcgen05 kernel with one tile's copy left out and a wait budget of a millisecond: the MMA role's wait
    for that tile runs out, every role drains, TMEM is freed, the kernel returns, and the status word reads
    CTB_ETIMEOUT.  A normal call right after is bit-exact: the context and the SM's tensor memory are intact."""
    from compressed_tensors_b200 import ops

    dev = torch.device("cuda", 0)
    sg = signs128(3).cuda()
    ws = [weights(256, 512, 70).cuda(), weights(128, 128, 71).cuda()]   # 8 + 1 tiles
    packed = [torch.empty((w.shape[0], w.shape[1] // 8), dtype=torch.int32, device=dev) for w in ws]
    scales = [torch.empty((w.shape[0], w.shape[1] // 128), dtype=torch.bfloat16, device=dev) for w in ws]
    table = ops.tensor_table(ws, packed, scales, [tuple(w.shape) for w in ws])
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    for skip in (0, 8):  # the first tile of a block's sequence, and the single tile of another block
        status.zero_()
        ops.rotate_quantize_int4_batch_bounded(table, sg, status, spin_cycles=2_000_000, skip_tile=skip, device=dev)
        torch.cuda.synchronize()
        assert int(status.item()) == 5, "CTB_ETIMEOUT"
    # no tile skipped, generous budget: a normal run through the same entry point
    status.zero_()
    ops.rotate_quantize_int4_batch_bounded(table, sg, status, spin_cycles=2_000_000_000, skip_tile=-1, device=dev)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    for w, p, s in zip(ws, packed, scales):
        gw, gs = ops.absmax_quantize(w, qtype=ops.QINT, bits=4, col_group=128, codec="pack32", hadamard_n=128, signs=sg,
                                     precision=ops.ROT_TENSOR)
        assert_bit_equal(p.cpu(), gw.cpu(), "words after a timed-out launch")
        assert_bit_equal(s.cpu(), gs.cpu(), "scales after a timed-out launch")


def test_engine_reports_a_device_timeout():
    """The engine hands the kernel a status word in page-locked host memory (no copy is needed to read it) and turns
    CTB_ETIMEOUT into TimeoutError at its next synchronisation point.  Driven end to end: the kernel itself writes the
    word when its wait runs out."""
    from compressed_tensors_b200 import ops
    from compressed_tensors_b200.compressors.model_compressors.engine import CodecEngine

    eng = CodecEngine()
    dev = torch.device("cuda", 0)
    word = eng._status_word(dev)
    assert word.is_pinned() and not word.is_cuda
    sg = signs128(3).cuda()
    w = weights(128, 128, 72).cuda()
    packed = torch.empty((128, 16), dtype=torch.int32, device=dev)
    scale = torch.empty((128, 1), dtype=torch.bfloat16, device=dev)
    table = ops.tensor_table([w], [packed], [scale], [(128, 128)])
    ops.rotate_quantize_int4_batch_bounded(table, sg, word, spin_cycles=2_000_000, skip_tile=0, device=dev)
    torch.cuda.synchronize()
    assert int(word[0]) == 5
    with pytest.raises(TimeoutError):
        eng.finish()
    eng.finish()  # the word was cleared


def test_sparse24_decompress_short_values_take_the_generic_kernels():
    """A bitmask with fewer than two bits per four has fewer values than the scan-free kernels would read: the entry
    point must route it to the kernels that read exactly `nnz` values.  The values live in an exact-size buffer
    between canary pages; the launch count shows which kernels ran."""
    from compressed_tensors_b200 import _lib as L
    from compressed_tensors_b200 import ops
    from oracle import ref as orc

    g = torch.Generator().manual_seed(3)
    w = weights(64, 512, 9)
    w[torch.rand(64, 512, generator=g) < 0.97] = 0     # 3 % dense
    values, bitmask, _ = orc.bitmask_compress(w)
    want = orc.bitmask_decompress(values, bitmask, w.shape)
    exact = values.clone().cuda()                         # holds nnz elements and nothing more
    assert exact.numel() < w.numel() // 2
    n0 = L.launch_count()
    got = ops.sparse24_decompress(exact, bitmask.cuda(), w.shape)
    torch.cuda.synchronize()
    assert L.launch_count() - n0 == 2, "two generic kernels, no scan-free launch in front"
    assert_bit_equal(got.cpu(), want, "short values")
    # a full-size buffer with a regular mask still takes the scan-free kernel (one launch + the gated fallback, which is one)
    t = weights(64, 512, 10)
    v, b = ops.sparse24_compress(t.cuda())
    n0 = L.launch_count()
    ops.sparse24_decompress(v, b, t.shape)
    assert L.launch_count() - n0 == 2


def test_sparse24_decompress_replayed_from_a_graph_with_changing_bitmasks():
    """One captured launch sequence, replayed over buffers whose contents change between replays: a two-per-four
    bitmask, then an irregular one (the gated fallback must run and give the generic codec's result), then a regular
    one again.  Nothing in the sequence may depend on state that a replay repeats (tickets, tags) for its result."""
    from compressed_tensors_b200 import ops
    from oracle import ref as orc

    orc.build()
    rows, cols = 96, 1024
    g = torch.Generator().manual_seed(5)

    def regular(seed):
        t = weights(rows, cols, seed)
        v, b = orc.sparse24_compress(t)
        return v.flatten(), b, orc.bitmask_decompress(v, b, t.shape)

    def irregular():
        t = weights(rows, cols, 77)
        t[torch.rand(rows, cols, generator=g) < 0.6] = 0  # fewer than two kept per four on average, unevenly spread
        v, b, _ = orc.bitmask_compress(t)
        room = torch.zeros(rows * cols // 2, dtype=t.dtype)  # a buffer of two per four, so the scan-free kernel runs first
        assert v.numel() <= room.numel()
        room[:v.numel()] = v
        return room, b, orc.bitmask_decompress(v, b, t.shape)

    cases = [regular(1), irregular(), regular(2), irregular(), regular(3)]
    values = torch.empty(rows * cols // 2, dtype=torch.bfloat16, device="cuda")
    bitmask = torch.empty((rows, cols // 8), dtype=torch.uint8, device="cuda")
    values.copy_(cases[0][0]), bitmask.copy_(cases[0][1])
    ops.sparse24_decompress(values, bitmask, (rows, cols))  # warm-up outside the capture
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            out = ops.sparse24_decompress(values, bitmask, (rows, cols))
    for i, (v, b, want) in enumerate(cases):
        values.copy_(v), bitmask.copy_(b)
        graph.replay()
        torch.cuda.synchronize()
        assert_bit_equal(out.cpu(), want, f"replay {i}")


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs in one process")
def test_one_process_two_devices():
    """The tensor-core entry point opts into its large dynamic shared memory per device: a process that drives a second
    GPU must get the same bits there."""
    from compressed_tensors_b200 import ops

    sg = signs128(4)
    w = weights(512, 1024, 80)
    outs = []
    for idx in (0, 1):
        dev = torch.device("cuda", idx)
        with torch.cuda.device(dev):
            gw, gs = ops.absmax_quantize(w.to(dev), qtype=ops.QINT, bits=4, col_group=128, codec="pack32", hadamard_n=128,
                                         signs=sg.to(dev), precision=ops.ROT_TENSOR)
            torch.cuda.synchronize(dev)
            outs.append((gw.cpu(), gs.cpu()))
    assert_bit_equal(outs[0][0], outs[1][0], "words on cuda:0 vs cuda:1")
    assert_bit_equal(outs[0][1], outs[1][1], "scales on cuda:0 vs cuda:1")
