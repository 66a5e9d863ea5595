"""Registration of quantization parameters on a module, with the reference's names and shapes
(quantization/lifecycle/initialize.py:60-143 initialize_module_for_quantization, :153-277 initialize_qparams).

The parameter bookkeeping and the wrapped quantized forward are mirrored: a compressed checkpoint can be loaded into,
and decompressed from, a module that carries `weight_scale`, `weight_zero_point`, `weight_global_scale`,
`weight_g_idx` of the right shape and dtype, and its forward fake-quantizes activations and weights through the CUDA
kernels (lifecycle/forward.py).  Observers and calibration are not part of this package.
"""
from typing import Optional, Tuple, Union

import torch
from torch.nn import Module, Parameter

from ..quant_args import ActivationOrdering, DynamicType, QuantizationArgs, QuantizationStrategy
from ..quant_config import QuantizationStatus
from ..quant_scheme import QuantizationScheme
from ..utils.helpers import is_fp4, strategy_cdiv

__all__ = ["initialize_module_for_quantization", "initialize_qparams"]

_QPARAM_SUFFIXES = ("_scale", "_zero_point", "_global_scale", "_g_idx")


def _device_of(module: Module) -> torch.device:
    for p in module.parameters(recurse=False):
        return p.device
    return torch.device("cpu")


def _register(module: Module, name: str, tensor: torch.Tensor) -> None:
    if hasattr(module, name):
        delattr(module, name)
    module.register_parameter(name, Parameter(tensor, requires_grad=False))


def initialize_module_for_quantization(module: Module, scheme: Optional[QuantizationScheme] = None,
                                       force_zero_point: bool = True) -> None:
    """Attach scales / zero points (/ global scale, g_idx) for every quantized side of `scheme` to `module`.
    Parameters of an earlier scheme that no longer apply are removed first."""
    scheme = scheme or getattr(module, "quantization_scheme", None)
    if scheme is None:
        return
    for name in [n for n, _ in module.named_parameters(recurse=False)]:
        if name.startswith(("input", "weight_", "output")) and name.endswith(_QPARAM_SUFFIXES):
            delattr(module, name)
    weight = getattr(module, "weight", None)
    if not isinstance(weight, torch.Tensor):
        return  # the weight gives the observed shapes and the dtype of the scales: nothing to size against
    if scheme.input_activations is not None:
        initialize_qparams(module, "input", scheme.input_activations, weight.shape[-1:], weight.dtype, force_zero_point)
    if scheme.weights is not None:
        initialize_qparams(module, "weight", scheme.weights, weight.shape, weight.dtype, force_zero_point)
    if scheme.output_activations is not None:
        initialize_qparams(module, "output", scheme.output_activations, weight.shape[:-1], weight.dtype, force_zero_point)
    # initialize.py:138-141: the forward acts on the call-time status; a re-initialised module wraps its plain forward again
    from .forward import wrap_module_forward_quantized

    plain = getattr(module, "_ctb_plain_forward", None)
    if plain is None:
        module._ctb_plain_forward = plain = module.forward
    module.forward = plain
    wrap_module_forward_quantized(module, scheme)
    module.quantization_scheme = scheme
    module.quantization_status = QuantizationStatus.INITIALIZED


def initialize_qparams(module: Module, base_name: str, quantization_args: QuantizationArgs,
                       observed_shape: Tuple[Union[int, None], ...], observed_dtype: torch.dtype,
                       force_zero_point: bool = True) -> None:
    """`<base_name>_scale` always (unless the quantization is dynamic), `<base_name>_global_scale` for
    TENSOR_GROUP, `<base_name>_g_idx` for group activation ordering, `<base_name>_zero_point` when asymmetric or
    forced.  Shapes follow the strategy; NVFP4 scales are e4m3, otherwise scales take the observed float dtype."""
    args, strategy, device = quantization_args, quantization_args.strategy, _device_of(module)
    if args.dynamic is True:
        return
    if strategy == QuantizationStrategy.TENSOR_GROUP:
        _register(module, f"{base_name}_global_scale", torch.empty(1, dtype=torch.float32, device=device))
    if args.dynamic == DynamicType.LOCAL:
        return

    if strategy == QuantizationStrategy.TENSOR:
        shape = (1,)
    elif strategy == QuantizationStrategy.TOKEN:
        raise ValueError("Cannot perform static token quantization")
    elif strategy == QuantizationStrategy.CHANNEL:
        if len(observed_shape) < 2:
            raise ValueError("Channel quant requires at least 2 observed dimensions")
        shape = (observed_shape[-2], 1)
    elif strategy in (QuantizationStrategy.GROUP, QuantizationStrategy.TENSOR_GROUP):
        if args.group_size is None or len(observed_shape) < 1:
            raise ValueError("Group quant requires a group size and at least 1 observed dimension")
        shape = (*observed_shape[:-1], strategy_cdiv(observed_shape[-1], args.group_size, strategy))
        if args.actorder == ActivationOrdering.GROUP:
            _register(module, f"{base_name}_g_idx", torch.full((observed_shape[-1],), -1, dtype=torch.int, device=device))
    elif strategy == QuantizationStrategy.BLOCK:
        if args.block_structure is None or len(observed_shape) < 2:
            raise ValueError("Block quant requires a block structure and at least 2 observed dimensions")
        shape = (strategy_cdiv(observed_shape[-2], args.block_structure[-2], strategy),
                 strategy_cdiv(observed_shape[-1], args.block_structure[-1], strategy))
    else:
        raise ValueError(f"Unknown or unsupported strategy {strategy}")

    if is_fp4(quantization_args=args):
        scale_dtype = zp_dtype = torch.float8_e4m3fn
    else:
        scale_dtype = observed_dtype if observed_dtype in (torch.float16, torch.bfloat16, torch.float32, torch.float64) else torch.bfloat16
        zp_dtype = args.pytorch_dtype()
    _register(module, f"{base_name}_scale", torch.empty(shape, dtype=scale_dtype, device=device))
    if force_zero_point or not args.symmetric:
        _register(module, f"{base_name}_zero_point", torch.zeros(shape, dtype=zp_dtype, device=device))
