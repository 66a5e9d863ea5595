"""`hadamard` transform factory (transform/factory/hadamard.py of the reference)."""
import math
from typing import Optional

import torch
from torch.nn import Module, Parameter

from ... import torch_ops as ops
from ..transform_args import TransformArgs, TransformLocation
from ..transform_scheme import TransformScheme
from ..utils.hadamard import deterministic_hadamard_matrix
from ..utils.matrix import get_transform_size
from .base import TransformBase, TransformFactory

__all__ = ["HadamardFactory", "HadamardTransform"]


@TransformFactory.register("hadamard")
class HadamardFactory(TransformFactory):
    def __init__(self, name: str, scheme: TransformScheme, seed: Optional[int] = None):
        super().__init__(name, scheme, seed)
        self._weights = {}
        self._perms = {}

    def create_transform(self, module: Module, args: TransformArgs) -> "HadamardTransform":
        size = get_transform_size(module, args.location, self.scheme.head_dim)
        # offline transforms are built in float64, like the reference (hadamard.py:57)
        precision = self.scheme.precision if args.is_online() else torch.float64
        key = (size, precision)
        if key not in self._weights:  # one matrix per size, shared by every module (hadamard.py:64)
            self._weights[key] = self._create_weight(size, torch.device("cpu"), torch.device("cpu"), precision)
        perm = None
        if self.scheme.randomize:  # hadamard.py:62: one permutation per weight, drawn after the weight
            if key not in self._perms:
                self._perms[key] = Parameter(torch.randperm(size, generator=self.generator), requires_grad=False)
            perm = self._perms[key]
        return HadamardTransform(self._weights[key], perm, self.scheme, args, type(module))

    def _create_weight(self, size: int, device, construct_device, precision: torch.dtype) -> Parameter:
        return Parameter(deterministic_hadamard_matrix(size, precision, construct_device), requires_grad=False)


class HadamardTransform(TransformBase):
    """Holds the +-1 matrix for inspection / serialisation; forward() runs the CUDA butterfly, which
    needs only the matrix's first column (the random signs)."""

    def __init__(self, weight: Parameter, perm, scheme: TransformScheme, args: TransformArgs, module_type: type):
        super().__init__()
        self.weight, self.perm, self.scheme, self.args, self.module_type = weight, perm, scheme, args, module_type
        self._signs = weight.data[:, 0].to(torch.int8)  # weight = diag(signs) @ H, column 0 of H is all ones
        self._scale = math.sqrt(weight.size(0))

    def forward(self, value: torch.Tensor) -> torch.Tensor:
        """hadamard.py:104-121: (apply_transform_weight(W_h, value.to(W_h.dtype)) / sqrt(n)).to(value.dtype).
        Weights rotate along their input (side 0) or output (side 1) dimension; activations (`input` / `output`)
        rotate along their last dimension, in blocks of the transform size."""
        location = TransformLocation(self.args.location)
        if location in (TransformLocation.Q_ATTN, TransformLocation.K_CACHE):
            raise NotImplementedError(f"{location.value} transforms are outside this package")
        embedding = self.module_type == torch.nn.Embedding
        if not (self.module_type == torch.nn.Linear or (embedding and not location.is_online())):
            raise NotImplementedError(f"Applying transforms to {self.module_type} {self.args.location} is not supported")
        acc = torch.float64 if self.weight.dtype == torch.float64 else torch.float32
        signs = self._signs.to(value.device)
        n = self.weight.size(0)
        # randomize (hadamard.py:104-108) applies M[perm][:, perm] = P M P^T: permute the transformed axis into the
        # matrix's index space, run the butterfly, permute back.  The permutation acts inside every block of n.
        perm = inv = None
        if self.perm is not None:
            perm = self.perm.data.to(value.device)
            inv = torch.empty_like(perm)
            inv[perm] = torch.arange(n, device=perm.device)
        # matrix.py:113-126: which product each location stands for.  Linear (y = x W.T): weight_input is value @ M.T,
        # weight_output is M.T @ value, activations are value @ M.  Embedding (y = x W): weight_input is M @ value and
        # weight_output is value @ M.  The kernel's side 1 computes M.T @ value and its side 0 value @ M.T; `inverse`
        # (M replaced by M.T) flips either.
        rows_side = location == (TransformLocation.WEIGHT_INPUT if embedding else TransformLocation.WEIGHT_OUTPUT)
        if rows_side:
            if perm is not None:
                value = value.reshape(-1, n, value.shape[-1])[:, inv, :].reshape(value.shape)
            out = ops.hadamard(value, n, signs=signs, inverse=bool(self.args.inverse) != embedding, side=1, precision=acc)
            return out if perm is None else out.reshape(-1, n, out.shape[-1])[:, perm, :].reshape(out.shape)
        transposed = bool(self.args.inverse) != (location.is_online() or embedding)
        flat = value.reshape(-1, value.shape[-1])
        if perm is not None:
            flat = flat.reshape(flat.shape[0], -1, n)[:, :, inv].reshape(flat.shape)
        out = ops.hadamard(flat.contiguous(), n, signs=signs, inverse=transposed, side=0, precision=acc)
        if perm is not None:
            out = out.reshape(out.shape[0], -1, n)[:, :, perm].reshape(out.shape)
        return out.reshape(value.shape)
