"""CUTLASS 2:4 semi-structured conversions on the GPU, with the reference's names
(utils/semi_structured_conversions.py:79 sparse_semi_structured_from_dense_cutlass, :216
sparse_semi_structured_to_dense_cutlass) for 16-bit dense dtypes (int16 metadata)."""
import torch

from .. import torch_ops as ops
from .._lib import on_gpu

__all__ = ["sparse_semi_structured_from_dense_cutlass", "sparse_semi_structured_to_dense_cutlass", "mask_creator"]


def sparse_semi_structured_from_dense_cutlass(dense: torch.Tensor):
    """dense [m, k] (f16 / bf16) -> (sparse [m, k/2], meta_reordered int16 [m, k/16])."""
    if dense.dim() != 2:
        raise RuntimeError(f"Expected 2-dimensional dense tensor, got {dense.dim()}-dimensional tensor")
    if dense.dtype not in (torch.float16, torch.bfloat16):
        raise RuntimeError(f"Invalid datatype {dense.dtype} of dense matrix")
    return ops.cutlass24_compress(on_gpu(dense))


def sparse_semi_structured_to_dense_cutlass(sparse: torch.Tensor, meta_reordered: torch.Tensor) -> torch.Tensor:
    """(sparse [m, k/2], meta_reordered int16 [m, k/16]) -> dense [m, k]."""
    return ops.cutlass24_decompress(on_gpu(sparse), on_gpu(meta_reordered))



def mask_creator(tensor: torch.Tensor) -> torch.Tensor:
    """semi_structured_conversions.py:313-342: a 2:4 keep mask (1.0 = keep, 0.0 = prune) over runs of four elements of
    the flattened tensor, by magnitude.  Runs with equal magnitudes follow the tie order of get_24_bytemasks (the
    reference's argsort leaves that order unspecified)."""
    if tensor.numel() % 4 != 0:
        raise ValueError(f"Tensor of size {tensor.shape} can't be evenly divided into 4 groups")
    return ops.sparse24_mask(tensor.detach()).to(torch.float32)
