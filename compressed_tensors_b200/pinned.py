"""A pool of page-locked host blocks for the results of the host <-> device pipeline.

torch's own page-locked allocator decides when a freed block may be handed out again from events it records at
the moment the block is freed.  A pipeline that enqueues a whole pass ahead of the GPU frees the previous
generation of buffers while copies that read them are still queued, so those blocks stay unavailable for the
rest of the pass and every pass ends up calling cudaHostAlloc again (a fifth of a second per 512 MiB while the
GPU is busy).  This pool knows the pipeline's own synchronisation points instead: a block whose tensors have all
died is parked, and becomes available at the next point where the owner has waited for the device
(`settle()`), which needs no CUDA call when a block is taken.

A block is handed out as a uint8 tensor over the page-locked memory; views of it may live in module
parameters for as long as the caller likes.  When the last of them dies the block comes back by itself.
"""
import ctypes
import threading
from typing import List

import torch

from . import _lib as L

__all__ = ["PinnedPool", "pool"]

_GRAIN = 16 << 20  # block sizes are multiples of this


class _Block:
    __slots__ = ("ptr", "nbytes")

    def __init__(self, nbytes: int):
        p = ctypes.c_void_p()
        L.check(L.lib().ctb_pinned_alloc(ctypes.c_int64(nbytes), ctypes.byref(p)))
        self.ptr, self.nbytes = p.value, nbytes

    def free(self) -> None:
        if self.ptr:
            L.lib().ctb_pinned_free(ctypes.c_void_p(self.ptr))
            self.ptr = 0


class _Lease:
    """Lives in the buffer object behind one handed-out tensor; its end of life returns the block."""

    __slots__ = ("block", "owner")

    def __init__(self, block: _Block, owner: "PinnedPool"):
        self.block, self.owner = block, owner

    def __del__(self):
        try:
            self.owner._park(self.block)
        except Exception:  # interpreter shutdown
            pass


class PinnedPool:
    def __init__(self):
        self._free: List[_Block] = []      # available now
        self._parked: List[_Block] = []    # every tensor died, but device work that touched them may still be queued
        self._lock = threading.Lock()
        self.allocated_bytes = 0
        self.allocations = 0

    def take(self, nbytes: int) -> torch.Tensor:
        """A uint8 tensor of exactly `nbytes` bytes of page-locked memory."""
        nbytes = max(int(nbytes), 1)
        want = (nbytes + _GRAIN - 1) // _GRAIN * _GRAIN
        block = None
        with self._lock:
            best = -1
            for i, b in enumerate(self._free):  # smallest block that is large enough and not wastefully large
                if b.nbytes >= want and b.nbytes <= 2 * want and (best < 0 or b.nbytes < self._free[best].nbytes):
                    best = i
            if best >= 0:
                block = self._free.pop(best)
        if block is None:
            block = _Block(want)
            self.allocated_bytes += want
            self.allocations += 1
        arr = (ctypes.c_uint8 * nbytes).from_address(block.ptr)
        arr._lease = _Lease(block, self)  # the array is what the tensor's storage keeps alive
        return torch.frombuffer(arr, dtype=torch.uint8)

    def _park(self, block: _Block) -> None:
        with self._lock:
            self._parked.append(block)

    def settle(self) -> None:
        """Call after the device has been waited for: parked blocks become available."""
        with self._lock:
            if self._parked:
                self._free.extend(self._parked)
                self._parked = []

    def has_parked(self) -> bool:
        return bool(self._parked)

    def trim(self) -> None:
        """Give the available blocks back to the system."""
        with self._lock:
            blocks, self._free = self._free, []
        for b in blocks:
            self.allocated_bytes -= b.nbytes
            b.free()


_pool = None


def pool() -> PinnedPool:
    """The process-wide pool."""
    global _pool
    if _pool is None:
        _pool = PinnedPool()
    return _pool
