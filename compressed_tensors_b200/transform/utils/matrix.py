"""Applying a transform matrix to a Linear weight (transform/utils/matrix.py:24-171 of the reference)."""
from typing import Optional, Tuple

import torch

from ... import torch_ops as ops
from ..transform_args import TransformLocation
from .hadamard import deterministic_hadamard_matrix, is_pow2

__all__ = ["get_transform_size", "apply_transform_weight", "hadamard_structure"]


def get_transform_size(module: torch.nn.Module, location: TransformLocation, head_dim: Optional[int] = None) -> int:
    """matrix.py:24-62."""
    location = TransformLocation(location)
    if isinstance(module, torch.nn.Linear):
        size = module.in_features if location in (TransformLocation.INPUT, TransformLocation.WEIGHT_INPUT) else module.out_features
    elif isinstance(module, torch.nn.Embedding):
        size = module.num_embeddings if location in (TransformLocation.INPUT, TransformLocation.WEIGHT_INPUT) else module.embedding_dim
    else:
        raise NotImplementedError(f"Transforms on {type(module)} are not supported")
    if head_dim is not None:
        if size % head_dim != 0:
            raise ValueError(f"{head_dim} must divide {size} for {type(module)} at {location}")
        size = head_dim
    return size


def hadamard_structure(weight: torch.Tensor) -> Tuple[torch.Tensor, bool]:
    """(signs, transposed) such that weight == diag(signs) @ H (transposed False) or H @ diag(signs)
    (transposed True), H the Sylvester matrix; raises if the matrix is not of that form."""
    n = weight.shape[0]
    if weight.ndim != 2 or weight.shape[1] != n or not is_pow2(n):
        raise NotImplementedError("only square power-of-two Hadamard transforms are built")
    h = deterministic_hadamard_matrix(n, weight.dtype, weight.device)
    col = weight[:, 0]
    if torch.equal(weight, col[:, None] * h):
        return col, False
    row = weight[0, :]
    if torch.equal(weight, h * row[None, :]):
        return row, True
    raise NotImplementedError("dense (non-Hadamard) transform matrices are outside this package")


def apply_transform_weight(transform_weight: torch.Tensor, value: torch.Tensor, location: TransformLocation,
                           module_type: type) -> torch.Tensor:
    """matrix.py:65-134 for Hadamard-structured transform weights on torch.nn.Linear: the raw
    (un-normalised) product, accumulated in float64 when either operand is float64."""
    assert transform_weight.shape[0] == transform_weight.shape[1]
    location = TransformLocation(location)
    if location.is_online():
        raise NotImplementedError("online (activation-side) transforms are outside this package")
    if module_type != torch.nn.Linear:
        raise NotImplementedError(f"Applying transforms to {module_type} {location} is not supported")
    signs, transposed = hadamard_structure(transform_weight)
    n = transform_weight.shape[0]
    side = 0 if location == TransformLocation.WEIGHT_INPUT else 1
    acc = torch.float64 if value.dtype == torch.float64 or transform_weight.dtype == torch.float64 else torch.float32
    v = value if value.dtype in (torch.bfloat16, torch.float16, torch.float32) else value.to(torch.float32)
    return ops.hadamard(v, n, signs=signs.to(torch.int8), inverse=transposed, side=side, precision=acc, normalize=False).to(value.dtype)
