"""QuantizationScheme and the preset table (quantization/quant_scheme.py:36-339 of the reference)."""
import warnings
from copy import deepcopy
from typing import List, Optional

from pydantic import BaseModel, ConfigDict, model_validator

from ..config import CompressionFormat
from .quant_args import DynamicType, QuantizationArgs, QuantizationStrategy, QuantizationType

__all__ = ["QuantizationScheme", "preset_name_to_scheme", "is_preset_scheme", "PRESET_SCHEMES"]

_ACT_STRATEGIES = (QuantizationStrategy.TOKEN, QuantizationStrategy.TENSOR, QuantizationStrategy.GROUP,
                   QuantizationStrategy.TENSOR_GROUP, QuantizationStrategy.ATTN_HEAD)


class QuantizationScheme(BaseModel):
    targets: List[str]
    weights: Optional[QuantizationArgs] = None
    input_activations: Optional[QuantizationArgs] = None
    output_activations: Optional[QuantizationArgs] = None
    format: Optional[str] = None

    model_config = ConfigDict(extra="forbid")

    @model_validator(mode="after")
    def _after(self):
        inputs, outputs, weights = self.input_activations, self.output_activations, self.weights
        if inputs is not None:
            if inputs.strategy not in _ACT_STRATEGIES:
                raise NotImplementedError(f"Using {inputs.strategy} strategy is not supported for activation quantization")
            if inputs.actorder is not None:
                raise ValueError("Cannot apply actorder to input activations")
        if outputs is not None and outputs.actorder is not None:
            raise ValueError("Cannot apply actorder to output activations")
        if self.format == CompressionFormat.mixed_precision.value:
            raise ValueError("mixed-precision cannot be set as a format for a QuantizationScheme")
        if (inputs and weights and weights.strategy == QuantizationStrategy.GROUP and inputs.strategy == QuantizationStrategy.GROUP
                and weights.group_size != inputs.group_size):
            warnings.warn("Using GROUP strategy for both weights and input_activations with different group sizes "
                          f"({weights.group_size} vs {inputs.group_size}) may complicate fused kernel implementations.",
                          UserWarning, stacklevel=2)
        return self


def _w(**kw):
    return QuantizationArgs(**kw)


INT, FLOAT = QuantizationType.INT, QuantizationType.FLOAT
S = QuantizationStrategy

PRESET_SCHEMES = {
    "UNQUANTIZED": dict(),
    "W8A16": dict(weights=_w(num_bits=8, type=INT, strategy=S.CHANNEL, symmetric=True, dynamic=False)),
    "W4A16": dict(weights=_w(num_bits=4, type=INT, strategy=S.GROUP, group_size=128, symmetric=True, dynamic=False)),
    "W4A16_ASYM": dict(weights=_w(num_bits=4, type=INT, strategy=S.GROUP, group_size=128, symmetric=False, dynamic=False)),
    "W8A8": dict(weights=_w(num_bits=8, type=INT, strategy=S.CHANNEL, symmetric=True, dynamic=False),
                 input_activations=_w(num_bits=8, type=INT, strategy=S.TOKEN, symmetric=True, dynamic=True, observer=None)),
    "INT8": dict(weights=_w(num_bits=8, type=INT, strategy=S.CHANNEL, symmetric=True, dynamic=False),
                 input_activations=_w(num_bits=8, type=INT, strategy=S.TOKEN, symmetric=True, dynamic=True, observer=None)),
    "W4A8": dict(weights=_w(num_bits=4, type=INT, strategy=S.GROUP, group_size=128, symmetric=True, dynamic=False),
                 input_activations=_w(num_bits=8, type=INT, strategy=S.TOKEN, symmetric=True, dynamic=True, observer=None)),
    "FP8": dict(weights=_w(num_bits=8, type=FLOAT, strategy=S.TENSOR, symmetric=True, dynamic=False),
                input_activations=_w(num_bits=8, type=FLOAT, strategy=S.TENSOR, symmetric=True, dynamic=False)),
    "FP8_DYNAMIC": dict(weights=_w(num_bits=8, type=FLOAT, strategy=S.CHANNEL, symmetric=True, dynamic=False),
                        input_activations=_w(num_bits=8, type=FLOAT, strategy=S.TOKEN, symmetric=True, dynamic=True, observer=None)),
    "FP8_BLOCK": dict(weights=_w(num_bits=8, type=FLOAT, strategy=S.BLOCK, symmetric=True, dynamic=False, block_structure=[128, 128]),
                      input_activations=_w(num_bits=8, type=FLOAT, strategy=S.GROUP, symmetric=True, dynamic=True, observer=None, group_size=128)),
    "NVFP4A16": dict(weights=_w(num_bits=4, type=FLOAT, strategy=S.TENSOR_GROUP, symmetric=True, dynamic=False, group_size=16)),
    "NVFP4": dict(weights=_w(num_bits=4, type=FLOAT, strategy=S.TENSOR_GROUP, symmetric=True, dynamic=False, group_size=16),
                  input_activations=_w(num_bits=4, type=FLOAT, strategy=S.TENSOR_GROUP, symmetric=True, dynamic=DynamicType.LOCAL, group_size=16)),
}


def preset_name_to_scheme(name: str, targets: List[str]) -> QuantizationScheme:
    name = name.upper()
    if name not in PRESET_SCHEMES:
        raise KeyError(f"Unknown preset scheme name {name}, available names: {list(PRESET_SCHEMES.keys())}")
    return QuantizationScheme(targets=targets, **deepcopy(PRESET_SCHEMES[name]))


def is_preset_scheme(name: str) -> bool:
    return name.upper() in PRESET_SCHEMES
