"""`random-hadamard` transform factory (transform/factory/random_hadamard.py of the reference)."""
import torch
from torch.nn import Parameter

from ..utils.hadamard import random_hadamard_matrix
from .base import TransformFactory
from .hadamard import HadamardFactory

__all__ = ["RandomHadamardFactory"]


@TransformFactory.register("random-hadamard")
class RandomHadamardFactory(HadamardFactory):
    def _create_weight(self, size: int, device, construct_device, precision: torch.dtype) -> Parameter:
        return Parameter(random_hadamard_matrix(size, precision, construct_device, self.generator), requires_grad=False)
