"""`sparse-24-bitmask`: 2:4 semi-structured values + packed bitmask
(compressors/sparse_compressors/sparse_24_bitmask.py of the reference)."""
from typing import Dict, List, Tuple, Union

import torch
from torch import Tensor

from ... import torch_ops as ops
from ..._lib import on_gpu
from ...config import CompressionFormat, SparsityStructure
from ...utils.helpers import merge_names
from ..base import BaseCompressor
from .base import BaseSparseCompressor

__all__ = ["Sparse24BitMaskCompressor", "Sparse24BitMaskTensor", "sparse24_bitmask_compress", "sparse24_bitmask_decompress", "get_24_bytemasks"]


def get_24_bytemasks(tensor: Tensor) -> Tensor:
    """sparse_24_bitmask.py:227-260: keep the two largest magnitudes of every run of four (flat view);
    e4m3 tensors are ranked through their int8 bit patterns; ties fall as torch.topk's do on CPU."""
    if tensor.numel() % 4 != 0:
        raise ValueError("Tensor size must be a multiple of 4 for TWO_FOUR sparsity")
    return ops.sparse24_mask(tensor)


def sparse24_bitmask_compress(tensor: Tensor, sparsity_structure: Union[SparsityStructure, str] = SparsityStructure.TWO_FOUR
                              ) -> Tuple[Tensor, Tensor]:
    """sparse_24_bitmask.py:162-203 -> (values [R, C/2], bitmask uint8 [R, ceil(C/8)])."""
    assert len(tensor.shape) == 2, "Only 2D tensors are supported"
    assert SparsityStructure(sparsity_structure) == SparsityStructure.TWO_FOUR, "Only 2:4 sparsity is supported"
    return ops.sparse24_compress(tensor)  # a torch operator with a fake implementation: meta tensors give meta results


def sparse24_bitmask_decompress(values: Tensor, bitmasks: Tensor, original_shape: torch.Size) -> Tensor:
    """sparse_24_bitmask.py:206-224."""
    shape = [int(s) for s in original_shape]
    return ops.sparse24_decompress(values.to(bitmasks.device), bitmasks, shape)


class Sparse24BitMaskTensor:
    def __init__(self, shape: Union[torch.Size, List], compressed: Tensor, bitmask: Tensor):
        self.shape = list(shape)
        self.compressed, self.bitmask = compressed, bitmask

    @staticmethod
    def from_dense(tensor: Tensor, sparsity_structure=SparsityStructure.TWO_FOUR) -> "Sparse24BitMaskTensor":
        compressed, bitmask = sparse24_bitmask_compress(tensor if tensor.is_meta else on_gpu(tensor), sparsity_structure=sparsity_structure)
        return Sparse24BitMaskTensor(shape=list(tensor.shape), compressed=compressed, bitmask=bitmask)

    @staticmethod
    def from_compressed_data(shape, compressed: Tensor, bitmask: Tensor) -> "Sparse24BitMaskTensor":
        if isinstance(shape, list):
            shape = torch.tensor(shape)
        if isinstance(shape, torch.Tensor):
            shape = shape.flatten().tolist()
        return Sparse24BitMaskTensor(shape=shape, compressed=compressed, bitmask=bitmask)

    def decompress(self) -> Tensor:
        return sparse24_bitmask_decompress(self.compressed, self.bitmask, self.shape)

    def curr_memory_size_bytes(self) -> int:
        return sum(t.element_size() * t.nelement() for t in (self.compressed, self.bitmask))

    def dict(self, name_prefix: str, device: str = "cpu") -> Dict[str, Tensor]:
        if name_prefix.endswith(".weight"):
            name_prefix = name_prefix[: -len(".weight")]
        return {
            merge_names(name_prefix, "shape"): torch.tensor(self.shape, device=device).reshape(-1, 1),
            merge_names(name_prefix, "compressed"): self.compressed.to(device),
            merge_names(name_prefix, "bitmask"): self.bitmask.to(device),
        }

    def __repr__(self) -> str:
        return f"BitMaskTensor(shape={self.shape}, compressed=True)"


@BaseCompressor.register(name=CompressionFormat.sparse_24_bitmask.value)
class Sparse24BitMaskCompressor(BaseSparseCompressor):
    @property
    def compression_param_names(self) -> Tuple[str]:
        return ("shape", "compressed", "bitmask")

    def compress_weight(self, name, value):
        structure = getattr(self.config, "sparsity_structure", SparsityStructure.TWO_FOUR.value) if self.config else SparsityStructure.TWO_FOUR.value
        return Sparse24BitMaskTensor.from_dense(value, structure).dict(name_prefix=name, device="cpu")

    def decompress_weight(self, weight_data):
        dev = weight_data["bitmask"].device if weight_data["bitmask"].is_cuda else torch.device("cuda")
        return Sparse24BitMaskTensor.from_compressed_data(shape=weight_data["shape"], compressed=weight_data["compressed"].to(dev),
                                                          bitmask=weight_data["bitmask"].to(dev)).decompress()
