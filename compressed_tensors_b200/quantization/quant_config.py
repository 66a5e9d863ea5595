"""QuantizationConfig / QuantizationStatus and the module-matching glue that attaches schemes and
min-max calibrated qparams to a model (quantization/quant_config.py, lifecycle/apply.py and
lifecycle/initialize.py of the reference, reduced to what the codec path needs)."""
import re
from enum import Enum
from typing import Dict, Iterable, List, Optional, Tuple, Union

import torch
from pydantic import BaseModel, ConfigDict, Field

from ..config import CompressionFormat
from .quant_args import QuantizationArgs, QuantizationStrategy
from .quant_scheme import QuantizationScheme, preset_name_to_scheme
from .utils.helpers import calculate_qparams, generate_gparam, is_fp4

__all__ = ["QuantizationStatus", "QuantizationConfig", "match_named_modules", "apply_quantization_config", "calibrate_weight_qparams"]


class QuantizationStatus(str, Enum):
    INITIALIZED = "initialized"
    CALIBRATION = "calibration"
    FROZEN = "frozen"
    COMPRESSED = "compressed"


class QuantizationConfig(BaseModel):
    config_groups: Dict[str, Union[QuantizationScheme, List[str]]]
    quant_method: str = "compressed-tensors"
    kv_cache_scheme: Optional[QuantizationArgs] = None
    format: Union[str, List[str]] = CompressionFormat.dense.value
    quantization_status: QuantizationStatus = QuantizationStatus.INITIALIZED
    global_compression_ratio: Optional[float] = None
    ignore: Optional[List[str]] = Field(default_factory=list)

    model_config = ConfigDict(extra="forbid")

    def model_post_init(self, __context):
        for name, group in list(self.config_groups.items()):
            if not isinstance(group, QuantizationScheme):  # {"W4A16": ["Linear"]} shorthand
                self.config_groups[name] = preset_name_to_scheme(name, group)


def _matches(name: str, module: torch.nn.Module, target: str) -> bool:
    if target.startswith("re:"):
        return re.match(target[3:], name) is not None
    return name == target or module.__class__.__name__ == target


def match_named_modules(model, targets: Iterable[str], ignore: Iterable[str] = ()) -> List[Tuple[str, torch.nn.Module]]:
    """Modules whose name, class name or `re:` pattern matches a target and no ignore entry (utils/match.py:40).
    `model` is a module, or a list of (name, module) pairs from an earlier walk over one."""
    targets, ignore = list(targets or []), list(ignore or [])
    out = []
    for name, module in (model.named_modules() if isinstance(model, torch.nn.Module) else model):
        if any(_matches(name, module, t) for t in targets) and not any(_matches(name, module, i) for i in ignore):
            out.append((name, module))
    return out


def apply_quantization_config(model: torch.nn.Module, config: QuantizationConfig) -> None:
    """Attach `quantization_scheme` / `quantization_status` to every targeted module (lifecycle/apply.py:112-183)."""
    for scheme in config.config_groups.values():
        for _, module in match_named_modules(model, scheme.targets, config.ignore):
            module.quantization_scheme = scheme
            module.quantization_status = QuantizationStatus.INITIALIZED


@torch.no_grad()
def calibrate_weight_qparams(module: torch.nn.Module) -> None:
    """Min-max calibration of a module's weight: registers `weight_scale`, `weight_zero_point` and, for
    NVFP4, `weight_global_scale`, shaped as lifecycle/initialize.py:155-280 shapes them."""
    from .. import torch_ops as ops

    args: QuantizationArgs = module.quantization_scheme.weights
    w = module.weight.data
    rows, cols = w.shape
    gs = None
    if args.strategy == QuantizationStrategy.TENSOR_GROUP:
        mn, mx = ops.minmax(w, rows, cols)
        gs = generate_gparam(mn.reshape(()), mx.reshape(()))
        module.register_parameter("weight_global_scale", torch.nn.Parameter(gs, requires_grad=False))
    if args.strategy in (QuantizationStrategy.GROUP, QuantizationStrategy.TENSOR_GROUP):
        mn, mx = ops.minmax(w, 1, args.group_size)
    elif args.strategy == QuantizationStrategy.CHANNEL:
        mn, mx = ops.minmax(w, 1, cols)
    elif args.strategy == QuantizationStrategy.TENSOR:
        mn, mx = ops.minmax(w, rows, cols)
        mn, mx = mn.reshape(()), mx.reshape(())
    elif args.strategy == QuantizationStrategy.BLOCK:
        bh, bw = args.block_structure
        mn, mx = ops.minmax(w, bh, bw)
    else:
        raise NotImplementedError(f"weight calibration for strategy {args.strategy}")
    scale, zp = calculate_qparams(mn, mx, args, global_scale=gs if is_fp4(args) else None)
    module.register_parameter("weight_scale", torch.nn.Parameter(scale, requires_grad=False))
    module.register_parameter("weight_zero_point", torch.nn.Parameter(zp, requires_grad=False))
    module.quantization_status = QuantizationStatus.FROZEN
