"""Bool-mask <-> bit-mask packing with the reference's signatures (utils/helpers.py:302-339), on the device."""
from typing import List

import torch

from .. import ops

__all__ = ["pack_bitmasks", "unpack_bitmasks", "merge_names"]


def pack_bitmasks(bytemasks: torch.Tensor) -> torch.Tensor:
    """[R, C] mask -> uint8 [R, ceil(C/8)], column 8k+j in bit j of byte k (numpy.packbits, little)."""
    return ops.pack_bitmasks(bytemasks)


def unpack_bitmasks(packed_bitmasks: torch.Tensor, original_shape: List[int]) -> torch.Tensor:
    """Inverse of pack_bitmasks: bool tensor of `original_shape`."""
    return ops.unpack_bitmasks(packed_bitmasks, list(original_shape))


def merge_names(parent_name: str, child_name: str) -> str:
    return child_name if not parent_name else f"{parent_name}.{child_name}"
