"""State-dict walk shared by the quantization compressors
(compressors/quantized_compressors/base.py:69-258 of the reference).  The per-weight work runs on the
GPU the weight lives on; results move to `compression_device` only at the end, as in the reference."""
from typing import Any, Dict, Generator, Optional, Tuple

import torch
from torch import Tensor

from ..._lib import on_gpu
from ...quantization.quant_args import QuantizationArgs, QuantizationStrategy
from ..base import BaseCompressor

__all__ = ["BaseQuantizationCompressor"]


def _nested(state_dict: Dict[str, Tensor], param_names) -> Dict[str, Dict[str, Tensor]]:
    """{module_path: {param_name: tensor}} for every key that ends in one of `param_names`."""
    out: Dict[str, Dict[str, Tensor]] = {}
    for key, value in state_dict.items():
        for p in param_names:
            if key == p or key.endswith("." + p):
                out.setdefault(key[: -len(p)].rstrip("."), {})[p] = value
                break
    return out


class BaseQuantizationCompressor(BaseCompressor):
    def compress(self, model_state: Dict[str, Tensor], names_to_scheme: Dict[str, Any], show_progress: bool = False,
                 compression_device: str = "cpu", **kwargs) -> Dict[str, Tensor]:
        out: Dict[str, Tensor] = {}
        for name in list(model_state.keys()):
            value = model_state[name]
            if name.endswith("weight"):
                prefix = name.removesuffix("weight")
                scale = model_state.get(prefix + "weight_scale")
                if scale is None:  # not a quantized weight
                    out[name] = value.to(compression_device)
                    continue
                module_path = prefix[:-1] if prefix.endswith(".") else prefix
                compressed = self.compress_weight(
                    weight=on_gpu(value), scale=on_gpu(scale), zero_point=on_gpu(model_state.get(prefix + "weight_zero_point")),
                    global_scale=on_gpu(model_state.get(prefix + "weight_global_scale")), g_idx=on_gpu(model_state.get(prefix + "weight_g_idx")),
                    quantization_args=names_to_scheme[module_path].weights, device=compression_device)
                for k, v in compressed.items():
                    out[prefix + k] = self._deliver(v, compression_device)
            else:
                if name.endswith("zero_point") and self._skip_zp(name, names_to_scheme):
                    continue
                out[name] = value.to(compression_device)
        return out

    def _skip_zp(self, name: str, names_to_scheme: Dict[str, Any]) -> bool:
        """Zero points of symmetric schemes, and those the pack compressor stores packed, are dropped."""
        from .pack_quantized import PackedQuantizationCompressor

        module_name, zp_name = name.rsplit(".", 1) if "." in name else ("", name)
        scheme = names_to_scheme[module_name]
        args = {"weight_zero_point": scheme.weights, "input_zero_point": scheme.input_activations,
                "output_zero_point": scheme.output_activations}[zp_name]
        packed = isinstance(self, PackedQuantizationCompressor) and args.strategy in (
            QuantizationStrategy.GROUP.value, QuantizationStrategy.CHANNEL.value)
        return args.symmetric or packed

    def decompress(self, path_to_model_or_tensors, names_to_scheme: Dict[str, Any], device: str = "cpu"):
        """A state dict, a safetensors file or a checkpoint folder -> (module path, {name: tensor}) with the dense
        `weight` added.  From disk (quantized_compressors/base.py:190-237 of the reference), each layer's packed
        tensors are opened straight onto the GPU and unpacked + dequantized there; `device` is where the results
        are left ("cpu" reproduces the reference's default, a CUDA device keeps them where they were computed)."""
        if isinstance(path_to_model_or_tensors, dict):
            yield from self.decompress_from_state_dict(path_to_model_or_tensors, names_to_scheme)
        else:
            yield from self._decompress_from_path(str(path_to_model_or_tensors), names_to_scheme, device)

    def _decompress_from_path(self, path: str, names_to_scheme: Dict[str, Any], device: str):
        from safetensors import safe_open

        from ...utils.safetensors_load import get_nested_weight_mappings

        gpu = torch.device(device) if torch.device(device).type == "cuda" else torch.device("cuda", torch.cuda.current_device())
        handles: Dict[str, Any] = {}
        try:
            for module_path, locations in get_nested_weight_mappings(path, self.compression_param_names).items():
                weight_data: Dict[str, Tensor] = {}
                for param_name, file in locations.items():
                    if file not in handles:
                        handles[file] = safe_open(file, framework="pt", device=str(gpu))
                    weight_data[param_name] = handles[file].get_tensor(module_path + "." + param_name if module_path else param_name)
                if "weight_scale" in weight_data and module_path in names_to_scheme:
                    weight_data["weight"] = self.decompress_weight(compressed_data=weight_data,
                                                                   quantization_args=names_to_scheme[module_path].weights)
                    yield module_path, {k: self._deliver(v, device) for k, v in weight_data.items()}
        finally:
            handles.clear()

    @staticmethod
    def _deliver(tensor: Tensor, device) -> Tensor:
        """Leave a result on `device`.  To the host it goes through page-locked memory (a pageable destination makes
        the driver stage the copy in small pieces, which is slower than the decompression itself); torch's host
        allocator recycles the page-locked blocks once the caller drops the tensors."""
        if torch.device(device).type != "cpu" or not tensor.is_cuda:
            return tensor.to(device)
        out = torch.empty(tensor.shape, dtype=tensor.dtype, pin_memory=True)
        out.copy_(tensor, non_blocking=True)
        torch.cuda.current_stream(tensor.device).synchronize()
        return out

    def decompress_module(self, module: torch.nn.Module) -> Optional[Tensor]:
        """Dense weight of one compressed leaf module (compressors/base.py:165-190 of the reference), or None when
        the module carries no weight scheme."""
        scheme = getattr(module, "quantization_scheme", None)
        if scheme is None or getattr(scheme, "weights", None) is None:
            return None
        device = next(module.parameters()).device
        data = {name: on_gpu(p.data) for name, p in module.named_parameters(recurse=False)}
        return self.decompress_weight(compressed_data=data, quantization_args=scheme.weights).to(device)

    def decompress_from_state_dict(self, state_dict: Dict[str, Tensor], names_to_scheme: Dict[str, Any]
                                   ) -> Generator[Tuple[str, Dict[str, Tensor]], None, None]:
        for module_path, weight_data in _nested(state_dict, self.compression_param_names).items():
            weight_data = {k: on_gpu(v) for k, v in weight_data.items()}
            if "weight_scale" in weight_data:
                weight_data["weight"] = self.decompress_weight(compressed_data=weight_data,
                                                               quantization_args=names_to_scheme[module_path].weights)
                yield module_path, weight_data

    def decompress_module_from_state_dict(self, prefix: str, state_dict: Dict[str, Tensor], scheme) -> Dict[str, Tensor]:
        local = {k.removeprefix(f"{prefix}."): v for k, v in state_dict.items()}
        if "weight_scale" in local:
            local["weight"] = self.decompress_weight(compressed_data={k: on_gpu(v) for k, v in local.items()},
                                                     quantization_args=scheme.weights)
        return {f"{prefix}.{k}": v for k, v in local.items()}

    def compress_weight(self, weight, scale, quantization_args: QuantizationArgs, zero_point=None, g_idx=None, device=None,
                        global_scale=None) -> Dict[str, Tensor]:
        raise NotImplementedError()

    def decompress_weight(self, compressed_data: Dict[str, Tensor], quantization_args: Optional[QuantizationArgs] = None) -> Tensor:
        raise NotImplementedError()
