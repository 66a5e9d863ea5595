"""CUTLASS 2:4 semi-structured conversions on the GPU, with the reference's names
(utils/semi_structured_conversions.py:79 sparse_semi_structured_from_dense_cutlass, :216
sparse_semi_structured_to_dense_cutlass) for 16-bit dense dtypes (int16 metadata)."""
import torch

from .. import ops
from .._lib import on_gpu

__all__ = ["sparse_semi_structured_from_dense_cutlass", "sparse_semi_structured_to_dense_cutlass"]


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

