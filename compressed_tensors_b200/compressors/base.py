"""Compressor base class and registry (compressors/base.py:30-202 of the reference)."""
from abc import ABC, abstractmethod
from typing import Dict, Generator, Optional, Tuple, Union

import torch
from torch import Tensor

from ..registry import RegistryMixin

__all__ = ["BaseCompressor"]


class BaseCompressor(RegistryMixin, ABC):
    """A compressor turns dense parameters into their on-disk form and back.  Subclasses register
    under a format name: ``BaseCompressor.register(name="pack-quantized")``."""

    def __init__(self, config=None):
        self.config = config

    def compression_param_info(self, weight_shape: torch.Size, quantization_args=None) -> Dict[str, Tuple[torch.Size, torch.dtype]]:
        raise NotImplementedError()

    @property
    @abstractmethod
    def compression_param_names(self) -> Tuple[str]:
        raise NotImplementedError()

    @abstractmethod
    def compress(self, model_state: Dict[str, Tensor], **kwargs) -> Dict[str, Tensor]:
        raise NotImplementedError()

    @abstractmethod
    def decompress(self, path_to_model_or_tensors, device: str = "cpu", **kwargs) -> Generator[Tuple[str, Tensor], None, None]:
        raise NotImplementedError()
