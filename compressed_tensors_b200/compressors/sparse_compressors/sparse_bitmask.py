"""`sparse-bitmask`: non-zero values + packed bitmask + row offsets
(compressors/sparse_compressors/sparse_bitmask.py of the reference), compressed and expanded on the GPU."""
from typing import Dict, List, Tuple, Union

import torch
from torch import Tensor

from ... import torch_ops as ops
from ..._lib import on_gpu
from ...config import CompressionFormat
from ...utils.helpers import merge_names
from ..base import BaseCompressor
from .base import BaseSparseCompressor

__all__ = ["BitmaskCompressor", "BitmaskTensor", "bitmask_compress", "bitmask_decompress"]


def bitmask_compress(tensor: Tensor) -> Tuple[Tensor, Tensor, Tensor]:
    """sparse_bitmask.py:131-149 -> (values [nnz] row-major, bitmask uint8 [R, ceil(C/8)], row_offsets int64 [R])."""
    if tensor.ndim != 2:
        tensor = tensor.reshape(-1, tensor.shape[-1])
    return ops.bitmask_compress(tensor)


def bitmask_decompress(values: Tensor, bitmasks: Tensor, original_shape: torch.Size) -> Tensor:
    """sparse_bitmask.py:152-169."""
    shape = [int(s) for s in original_shape]
    rows = 1
    for s in shape[:-1]:
        rows *= s
    return ops.bitmask_decompress(values.to(bitmasks.device), bitmasks, (rows, shape[-1])).reshape(shape)


class BitmaskTensor:
    def __init__(self, shape: Union[torch.Size, List], compressed: Tensor, bitmask: Tensor, row_offsets: Tensor):
        self.shape = list(shape)
        self.compressed, self.bitmask, self.row_offsets = compressed, bitmask, row_offsets

    @staticmethod
    def from_dense(tensor: Tensor) -> "BitmaskTensor":
        compressed, bitmask, row_offsets = bitmask_compress(on_gpu(tensor))
        return BitmaskTensor(shape=tensor.shape, compressed=compressed, bitmask=bitmask, row_offsets=row_offsets)

    def decompress(self) -> Tensor:
        return bitmask_decompress(self.compressed, self.bitmask, self.shape)

    def curr_memory_size_bytes(self) -> int:
        return sum(t.element_size() * t.nelement() for t in (self.compressed, self.bitmask, self.row_offsets))

    def dict(self, name_prefix: str, device: str = "cpu") -> Dict[str, Tensor]:
        return {
            merge_names(name_prefix, "shape"): torch.tensor(self.shape, device=device),
            merge_names(name_prefix, "compressed"): self.compressed.to(device),
            merge_names(name_prefix, "bitmask"): self.bitmask.to(device),
            merge_names(name_prefix, "row_offsets"): self.row_offsets.to(device),
        }

    def __repr__(self):
        return f"BitmaskTensor(shape={self.shape}, compressed=True)"


@BaseCompressor.register(name=CompressionFormat.sparse_bitmask.value)
class BitmaskCompressor(BaseSparseCompressor):
    @property
    def compression_param_names(self) -> Tuple[str]:
        return ("shape", "compressed", "bitmask", "row_offsets")

    def compress_weight(self, name, value):
        return BitmaskTensor.from_dense(value).dict(name_prefix=name, device="cpu")

    def decompress_weight(self, weight_data):
        data = {k: v for k, v in weight_data.items()}
        data["shape"] = [int(s) for s in data["shape"].flatten().tolist()]
        dev = data["bitmask"].device if data["bitmask"].is_cuda else torch.device("cuda")
        return BitmaskTensor(shape=data["shape"], compressed=data["compressed"].to(dev), bitmask=data["bitmask"].to(dev),
                             row_offsets=data["row_offsets"]).decompress()
