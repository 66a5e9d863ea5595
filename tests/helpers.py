"""Shared comparison helpers for the parity tests."""
import torch


def bits_of(t: torch.Tensor) -> torch.Tensor:
    """Raw storage of a tensor as integers, for bit-exact comparison of any dtype."""
    t = t.detach().cpu().contiguous()
    if t.dtype == torch.bool:
        return t.to(torch.uint8)
    view = {1: torch.uint8, 2: torch.int16, 4: torch.int32, 8: torch.int64}[t.element_size()]
    return t.view(view)


def assert_bit_equal(a: torch.Tensor, b: torch.Tensor, what: str = "") -> None:
    assert a.dtype == b.dtype, f"{what}: dtype {a.dtype} vs {b.dtype}"
    assert tuple(a.shape) == tuple(b.shape), f"{what}: shape {tuple(a.shape)} vs {tuple(b.shape)}"
    ba, bb = bits_of(a), bits_of(b)
    if not torch.equal(ba, bb):
        bad = (ba != bb).flatten().nonzero().flatten()
        i = int(bad[0])
        raise AssertionError(
            f"{what}: {bad.numel()} of {ba.numel()} elements differ; first at flat index {i}: "
            f"{a.flatten()[i].item()!r} vs {b.flatten()[i].item()!r}"
        )


def assert_value_equal(a: torch.Tensor, b: torch.Tensor, what: str = "") -> None:
    """Equal as numbers (so -0.0 == 0.0), NaNs in the same places."""
    assert a.dtype == b.dtype and tuple(a.shape) == tuple(b.shape), what
    af, bf = a.double().cpu(), b.double().cpu()
    assert torch.equal(af.isnan(), bf.isnan()), what
    assert torch.equal(af.nan_to_num(), bf.nan_to_num()), what


def bf16_ulp_distance(a: torch.Tensor, b: torch.Tensor) -> int:
    """Largest distance, in bf16 steps, between two bf16 tensors (sign-magnitude aware)."""
    def key(t):
        v = t.detach().cpu().contiguous().view(torch.int16).to(torch.int32)
        return torch.where(v < 0, -(v & 0x7FFF), v)
    return int((key(a) - key(b)).abs().max())
