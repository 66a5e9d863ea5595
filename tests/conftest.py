import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def golden():
    import torch

    gdir = os.path.join(ROOT, "tests", "golden")

    def load(name):
        return torch.load(os.path.join(gdir, name + ".pt"), weights_only=True)

    return load


@pytest.fixture
def canary():
    """`with canary():` -- every CUDA tensor that compressed_tensors_b200.ops allocates inside the block sits between
    two 256-byte pages of a known pattern; on exit the device is synchronised and every page must be untouched.
    Stands in for a memory checker: a kernel that writes outside its output fails the test even when the output is
    right."""
    import contextlib
    import math

    import torch

    from compressed_tensors_b200 import ops

    PAD, PATTERN = 256, 0xA5

    class Proxy:
        def __init__(self, log):
            self._log = log

        def __getattr__(self, name):
            return getattr(torch, name)

        def _padded(self, shape, dtype, device):
            shape = tuple(int(s) for s in shape)
            nbytes = math.prod(shape) * torch.empty((), dtype=dtype).element_size()
            buf = torch.full((nbytes + 2 * PAD,), PATTERN, dtype=torch.uint8, device=device)
            self._log.append((buf, nbytes))
            return buf[PAD:PAD + nbytes].view(dtype).view(shape)

        def empty(self, *size, dtype=None, device=None, **kw):
            if device is None or torch.device(device).type != "cuda" or kw.get("pin_memory"):
                return torch.empty(*size, dtype=dtype, device=device, **kw)
            shape = size[0] if len(size) == 1 and isinstance(size[0], (tuple, list, torch.Size)) else size
            return self._padded(shape, dtype or torch.get_default_dtype(), device)

        def empty_like(self, t, **kw):
            if not t.is_cuda:
                return torch.empty_like(t, **kw)
            return self._padded(t.shape, kw.get("dtype", t.dtype), t.device)

    @contextlib.contextmanager
    def guard():
        log = []
        real = ops.torch
        ops.torch = Proxy(log)
        try:
            yield
        finally:
            ops.torch = real
        torch.cuda.synchronize()
        for buf, nbytes in log:
            head, tail = buf[:PAD], buf[PAD + nbytes:]
            assert bool((head == PATTERN).all()) and bool((tail == PATTERN).all()), \
                f"a kernel wrote outside an output of {nbytes} bytes"

    return guard
