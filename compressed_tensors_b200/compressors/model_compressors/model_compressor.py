"""Whole-model compress / decompress (compressors/model_compressors/model_compressor.py:87-920 of the
reference, the in-memory paths).  Same order of operations -- quantization compressor first, sparsity
compressor second on compress, the reverse on decompress -- and the same state-dict key contract; the
per-tensor work runs on the GPU that holds the module's weight.  Disk I/O (safetensors, config.json)
stays with the caller."""
from typing import Dict, List, Optional, Union

import torch
from torch.nn import Module

from ...config import CompressionFormat, SparsityCompressionConfig
from ...quantization.quant_config import QuantizationConfig, QuantizationStatus, match_named_modules
from ...quantization.quant_scheme import QuantizationScheme
from ..base import BaseCompressor

__all__ = ["ModelCompressor", "map_module_to_scheme"]


def map_module_to_scheme(model: Module) -> Dict[str, QuantizationScheme]:
    """{module name: scheme} for every module that carries a weight scheme (model_compressor.py:896-920)."""
    out = {}
    for name, module in model.named_modules():
        scheme = getattr(module, "quantization_scheme", None)
        if scheme is not None and (scheme.weights is not None or scheme.input_activations is not None):
            out[name] = scheme
    return out


class ModelCompressor:
    def __init__(self, sparsity_config: Optional[SparsityCompressionConfig] = None,
                 quantization_config: Optional[QuantizationConfig] = None, transform_config=None,
                 compression_formats: Optional[List[str]] = None):
        self.sparsity_config = sparsity_config
        self.quantization_config = quantization_config
        self.transform_config = transform_config
        self.compression_formats = compression_formats
        self.sparsity_compressor = None
        self.quantization_compressor: Optional[Dict[str, BaseCompressor]] = None
        if sparsity_config is not None:
            self.sparsity_compressor = BaseCompressor.load_from_registry(sparsity_config.format, config=sparsity_config)
        if quantization_config is not None:
            if not self.compression_formats:
                fmt = quantization_config.format
                self.compression_formats = list(fmt) if isinstance(fmt, (list, tuple)) else [fmt]
            self.quantization_compressor = {
                f: BaseCompressor.load_from_registry(f, config=quantization_config) for f in self.compression_formats
            }

    # ------------------------------------------------------------------ helpers
    def _format_for(self, scheme: QuantizationScheme) -> str:
        if getattr(scheme, "format", None):
            return scheme.format
        if len(self.compression_formats) > 1:
            raise ValueError("Applying multiple compressors without defining per module formats is not supported ")
        return self.compression_formats[0]

    def _sparse_targets(self, model: Module) -> List[str]:
        if self.sparsity_config is None:
            return []
        return [n for n, _ in match_named_modules(model, self.sparsity_config.targets or [], self.sparsity_config.ignore or [])]

    # ------------------------------------------------------------------ state-dict path
    def compress(self, model: Module, state_dict: Optional[Dict[str, torch.Tensor]] = None, show_progress: bool = False
                 ) -> Dict[str, torch.Tensor]:
        """model_compressor.py:621-674: returns the compressed state dict (tensors on the CPU, as the
        reference leaves them); the model itself is not modified."""
        if state_dict is None:
            state_dict = model.state_dict()
        if self.quantization_compressor is not None:
            module_to_scheme = map_module_to_scheme(model)
            by_format: Dict[str, Dict[str, torch.Tensor]] = {}
            rest: Dict[str, torch.Tensor] = {}
            for key, value in state_dict.items():
                module_name = key.rsplit(".", 1)[0] if "." in key else ""
                if module_name in module_to_scheme:
                    by_format.setdefault(self._format_for(module_to_scheme[module_name]), {})[key] = value
                else:
                    rest[key] = value
            merged: Dict[str, torch.Tensor] = {}
            for fmt, part in by_format.items():
                merged.update(self.quantization_compressor[fmt].compress(part, names_to_scheme=module_to_scheme,
                                                                         show_progress=show_progress, compression_device="cpu"))
            merged.update({k: v.to("cpu") for k, v in rest.items()})
            # keep the original key order where a key survived
            state_dict = {**{k: merged[k] for k in state_dict if k in merged}, **{k: v for k, v in merged.items() if k not in state_dict}}
        if self.sparsity_compressor is not None:
            targets = set(self._sparse_targets(model))
            state_dict = self.sparsity_compressor.compress(state_dict, compression_targets=targets, show_progress=show_progress)
        return state_dict

    # ------------------------------------------------------------------ in-place paths
    @torch.no_grad()
    def compress_model(self, model: Module) -> None:
        """model_compressor.py:453-539: replace each targeted module's parameters by their compressed form."""
        module_to_scheme = map_module_to_scheme(model)
        sparse_targets = self._sparse_targets(model)
        names = list(dict.fromkeys([*sparse_targets, *module_to_scheme.keys()]))
        modules = dict(model.named_modules())
        for prefix in names:
            module = modules[prefix]
            device = next(module.parameters(recurse=False)).device
            state = {f"{prefix}.{n}": p.data for n, p in module.named_parameters(recurse=False)}
            if prefix in module_to_scheme and self.quantization_compressor is not None:
                comp = self.quantization_compressor[self._format_for(module_to_scheme[prefix])]
                state = comp.compress(state, names_to_scheme=module_to_scheme, show_progress=False, compression_device=device)
            if prefix in sparse_targets:
                state = self.sparsity_compressor.compress(state, compression_targets=set(sparse_targets), show_progress=False)
            for n, _ in list(module.named_parameters(recurse=False)):
                delattr(module, n)
            for n, v in state.items():
                module.register_parameter(n.removeprefix(f"{prefix}."), torch.nn.Parameter(v.to(device), requires_grad=False))
            module.quantization_status = QuantizationStatus.COMPRESSED
        if self.quantization_config is not None and self.quantization_config.format != CompressionFormat.dense.value:
            self.quantization_config.quantization_status = QuantizationStatus.COMPRESSED

    @torch.no_grad()
    def decompress_model(self, model: Module) -> None:
        """model_compressor.py:541-617: sparsity decompression first, then quantization decompression."""
        module_to_scheme = map_module_to_scheme(model)
        sparse_targets = self._sparse_targets(model)
        names = list(dict.fromkeys([*sparse_targets, *module_to_scheme.keys()]))
        modules = dict(model.named_modules())
        for prefix in names:
            module = modules[prefix]
            device = next(module.parameters(recurse=False)).device
            state = {f"{prefix}.{n}": p.data for n, p in module.named_parameters(recurse=False)}
            if prefix in sparse_targets and self.sparsity_compressor is not None:
                state = dict(self.sparsity_compressor.decompress_from_state_dict(state)) | {
                    k: v for k, v in state.items() if k.rsplit(".", 1)[-1] not in self.sparsity_compressor.compression_param_names}
            if prefix in module_to_scheme and self.quantization_compressor is not None:
                comp = self.quantization_compressor[self._format_for(module_to_scheme[prefix])]
                state = comp.decompress_module_from_state_dict(prefix, state, scheme=module_to_scheme[prefix])
            for n, _ in list(module.named_parameters(recurse=False)):
                delattr(module, n)
            drop = ("weight_packed", "weight_shape", "compressed", "bitmask", "shape", "row_offsets")
            for n, v in state.items():
                short = n.removeprefix(f"{prefix}.")
                if short in drop:
                    continue
                module.register_parameter(short, torch.nn.Parameter(v.to(device), requires_grad=False))
            module.quantization_status = QuantizationStatus.FROZEN
