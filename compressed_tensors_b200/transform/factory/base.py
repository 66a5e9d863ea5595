"""TransformFactory / TransformBase (transform/factory/base.py of the reference): the fuse-into-weight
locations and the activation-side `input` / `output` hooks.  The attention locations (`q_attn`, `k_cache`) hook
into a transformers model and are outside this package."""
from abc import ABC, abstractmethod
from typing import Optional

import torch
from torch.nn import Module, Parameter

from ...quantization.quant_config import match_named_modules
from ...registry import RegistryMixin
from ..transform_args import TransformArgs, TransformLocation
from ..transform_scheme import TransformScheme

__all__ = ["TransformFactory", "TransformBase"]


class TransformBase(Module, ABC):
    args: TransformArgs
    weight: Parameter

    @abstractmethod
    def forward(self, value: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError()


class TransformFactory(RegistryMixin, ABC):
    def __init__(self, name: str, scheme: TransformScheme, seed: Optional[int] = None):
        self.name, self.scheme = name, scheme
        self.generator = torch.Generator()
        if seed is not None:
            self.generator.manual_seed(seed)

    @classmethod
    def from_scheme(cls, scheme: TransformScheme, **kwargs):
        return cls.get_value_from_registry(scheme.type)(scheme=scheme, **kwargs)

    @abstractmethod
    def create_transform(self, module: Module, args: TransformArgs) -> TransformBase:
        raise NotImplementedError()

    def apply_to_model(self, model: Module) -> None:
        """base.py:95-109: every (module, args) pair matched by the scheme."""
        for args in self.scheme.apply:
            for _, module in match_named_modules(model, args.targets, args.ignore):
                self._apply_to_module(module, args)

    def _apply_to_module(self, module: Module, args: TransformArgs) -> None:
        """base.py:111-192.  weight_input / weight_output: rotate the weight once and keep no submodule.
        input / output: keep the transform as a submodule and run it on the activations through a forward
        (pre-)hook."""
        location = TransformLocation(args.location)
        transform = self.create_transform(module, args)
        if location in (TransformLocation.WEIGHT_INPUT, TransformLocation.WEIGHT_OUTPUT):
            with torch.no_grad():
                module.weight.data = transform(module.weight.data)
            return
        if location not in (TransformLocation.INPUT, TransformLocation.OUTPUT):
            raise NotImplementedError(f"{location.value} transforms hook into a transformers attention module: outside this package")
        module.add_module(f"{self.name}_{location.value}", transform)
        if location == TransformLocation.INPUT:
            module.register_forward_pre_hook(lambda _, inputs: transform(inputs[0]), prepend=True)
        else:
            module.register_forward_hook(lambda _, _inputs, output: transform(output))
