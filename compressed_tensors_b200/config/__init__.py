"""Format names and sparsity configuration (config/base.py:25-114 of the reference)."""
from enum import Enum, unique
from typing import List, Optional

from pydantic import BaseModel

from ..registry import RegistryMixin

__all__ = ["CompressionFormat", "SparsityStructure", "SparsityCompressionConfig", "BitmaskConfig", "Sparse24BitMaskConfig", "DenseSparsityConfig"]


@unique
class CompressionFormat(Enum):
    dense = "dense"
    sparse_bitmask = "sparse-bitmask"
    sparse_24_bitmask = "sparse-24-bitmask"
    int_quantized = "int-quantized"
    float_quantized = "float-quantized"
    naive_quantized = "naive-quantized"
    pack_quantized = "pack-quantized"
    marlin_24 = "marlin-24"
    mixed_precision = "mixed-precision"
    nvfp4_pack_quantized = "nvfp4-pack-quantized"
    mxfp4_pack_quantized = "mxfp4-pack-quantized"


@unique
class SparsityStructure(Enum):
    TWO_FOUR = "2:4"
    UNSTRUCTURED = "unstructured"
    ZERO_ZERO = "0:0"

    def __new__(cls, value):
        obj = object.__new__(cls)
        obj._value_ = value.lower()
        return obj

    @classmethod
    def _missing_(cls, value):
        if value is None:
            return cls.UNSTRUCTURED
        for member in cls:
            if member.value == str(value).lower():
                return member
        raise ValueError(f"{value} is not a valid {cls.__name__}")


class SparsityCompressionConfig(RegistryMixin, BaseModel):
    format: str
    targets: Optional[List[str]] = None
    ignore: Optional[List[str]] = None
    global_sparsity: Optional[float] = 0.0
    sparsity_structure: Optional[str] = "unstructured"


@SparsityCompressionConfig.register(name=CompressionFormat.sparse_bitmask.value)
class BitmaskConfig(SparsityCompressionConfig):
    format: str = CompressionFormat.sparse_bitmask.value


@SparsityCompressionConfig.register(name=CompressionFormat.sparse_24_bitmask.value)
class Sparse24BitMaskConfig(SparsityCompressionConfig):
    format: str = CompressionFormat.sparse_24_bitmask.value
    sparsity_structure: Optional[str] = SparsityStructure.TWO_FOUR.value


@SparsityCompressionConfig.register(name=CompressionFormat.dense.value)
class DenseSparsityConfig(SparsityCompressionConfig):
    format: str = CompressionFormat.dense.value
