"""State-dict walk of the sparsity compressors (compressors/sparse_compressors/base.py:66-176)."""
from typing import Dict, Generator, Optional, Set, Tuple

from torch import Tensor

from ...utils.helpers import merge_names
from ..base import BaseCompressor

__all__ = ["BaseSparseCompressor"]


class BaseSparseCompressor(BaseCompressor):
    def compress(self, model_state: Dict[str, Tensor], compression_targets: Optional[Set[str]] = None,
                 show_progress: bool = False) -> Dict[str, Tensor]:
        out: Dict[str, Tensor] = {}
        for name, value in model_state.items():
            if not self.should_compress(name, compression_targets):
                out[name] = value
                continue
            prefix = name.removesuffix(".weight") if name.endswith(".weight") else name
            for key, v in self.compress_weight(prefix, value).items():
                if key in out:
                    raise ValueError(f"Expected all compressed state_dict keys to be unique, but found an existing entry for {key}.")
                out[key] = v
        return out

    def decompress(self, path_to_model_or_tensors, device: str = "cpu", **kwargs):
        if not isinstance(path_to_model_or_tensors, dict):
            raise NotImplementedError("reading safetensors from disk is outside this package; pass a state dict")
        yield from self.decompress_from_state_dict(path_to_model_or_tensors)

    def decompress_from_state_dict(self, state_dict: Dict[str, Tensor]) -> Generator[Tuple[str, Tensor], None, None]:
        groups: Dict[str, Dict[str, Tensor]] = {}
        passthrough = []
        for key, value in state_dict.items():
            for p in self.compression_param_names:
                if key.endswith("." + p):
                    groups.setdefault(key[: -len(p) - 1], {})[p] = value
                    break
            else:
                passthrough.append((key, value))
        for prefix, data in groups.items():
            yield merge_names(prefix, "weight"), self.decompress_weight(data)
        for key, value in passthrough:
            if not key.endswith(".weight"):
                yield key, value

    @staticmethod
    def should_compress(name: str, expanded_targets: Optional[Set[str]] = None) -> bool:
        if expanded_targets is None:
            return name.endswith(".weight")
        return name.endswith(".weight") and name[: -len(".weight")] in expanded_targets
