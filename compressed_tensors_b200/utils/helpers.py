"""Bool-mask <-> bit-mask packing with the reference's signatures (utils/helpers.py:302-339), on the device."""
from typing import List

import torch

from .. import torch_ops as ops

__all__ = ["pack_bitmasks", "unpack_bitmasks", "merge_names", "tensor_follows_mask_structure"]


def pack_bitmasks(bytemasks: torch.Tensor) -> torch.Tensor:
    """[R, C] mask -> uint8 [R, ceil(C/8)], column 8k+j in bit j of byte k (numpy.packbits, little)."""
    return ops.pack_bitmasks(bytemasks)


def unpack_bitmasks(packed_bitmasks: torch.Tensor, original_shape: List[int]) -> torch.Tensor:
    """Inverse of pack_bitmasks: bool tensor of `original_shape`."""
    return ops.unpack_bitmasks(packed_bitmasks, list(original_shape))


def merge_names(parent_name: str, child_name: str) -> str:
    return child_name if not parent_name else f"{parent_name}.{child_name}"


def tensor_follows_mask_structure(tensor: torch.Tensor, mask: str = "2:4") -> bool:
    """utils/helpers.py:93-115: True when every run of m elements holds at least n zeros (some weights may be zero by
    chance, hence "at least"); raises ValueError otherwise, like the reference."""
    n, m = (int(v) for v in mask.split(":"))
    zeros = (tensor.reshape(-1, m) == 0).sum(dim=1)
    if not bool((zeros >= n).all()):
        raise ValueError()
    return True
