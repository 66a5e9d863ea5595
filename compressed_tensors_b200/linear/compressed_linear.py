"""A Linear that holds its weight compressed and decompresses it on the GPU at its first forward
(linear/compressed_linear.py:33-109 of the reference: same construction through `from_linear`, same parameter
names, same status transitions COMPRESSED -> FROZEN)."""
import warnings
from typing import Dict, Tuple

import torch
from torch import Tensor
from torch.nn import Parameter
from torch.nn.functional import linear
from torch.nn.modules import Linear

from ..compressors.base import BaseCompressor
from ..quantization.lifecycle.initialize import initialize_module_for_quantization
from ..quantization.quant_config import QuantizationStatus
from ..quantization.quant_scheme import QuantizationScheme

__all__ = ["CompressedLinear"]


class CompressedLinear(Linear):
    def __init__(self, *args, **kwargs) -> None:
        super().__init__(*args, **kwargs)
        warnings.warn("CompressedLinear should not be initialized directly. Use the from_linear method instead.", UserWarning)

    @classmethod
    @torch.no_grad()
    def from_linear(cls, module: Linear, quantization_scheme: QuantizationScheme, quantization_format: str):
        """Turn `module` into a CompressedLinear in place: register the scheme's scales / zero points and the
        format's compressed parameters (empty, to be filled by a checkpoint load) and drop the dense weight."""
        module.__class__ = CompressedLinear
        module.compressor = BaseCompressor.load_from_registry(quantization_format)
        device = module.weight.device
        initialize_module_for_quantization(module, quantization_scheme, force_zero_point=False)
        info: Dict[str, Tuple] = module.compressor.compression_param_info(module.weight.shape, quantization_scheme.weights)
        delattr(module, "weight")
        for name, (shape, dtype) in info.items():
            module.register_parameter(name, Parameter(torch.empty(shape, device=device, dtype=dtype), requires_grad=False))
        module.quantization_status = QuantizationStatus.COMPRESSED
        return module

    def forward(self, input: Tensor) -> Tensor:
        """Decompress once (unpack + dequantize kernels), keep the dense weight, then the ordinary linear."""
        if self.quantization_status == QuantizationStatus.COMPRESSED:
            self.register_parameter("weight", Parameter(self.compressor.decompress_module(self), requires_grad=False))
            self.quantization_status = QuantizationStatus.FROZEN
        return linear(input, self.weight, self.bias)
