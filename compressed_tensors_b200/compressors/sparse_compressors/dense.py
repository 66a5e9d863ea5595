"""`dense`: the identity compressor (compressors/sparse_compressors/dense.py of the reference)."""
from typing import Dict, Generator, Tuple

from torch import Tensor

from ...config import CompressionFormat
from ..base import BaseCompressor

__all__ = ["DenseCompressor"]


@BaseCompressor.register(name=CompressionFormat.dense.value)
class DenseCompressor(BaseCompressor):
    @property
    def compression_param_names(self) -> Tuple[str]:
        return ()

    def compress(self, model_state: Dict[str, Tensor], **kwargs) -> Dict[str, Tensor]:
        return model_state

    def decompress(self, path_to_model_or_tensors, device: str = "cpu", **kwargs) -> Generator[Tuple[str, Tensor], None, None]:
        return iter([])

    def decompress_from_state_dict(self, state_dict: Dict[str, Tensor]):
        yield from state_dict.items()
