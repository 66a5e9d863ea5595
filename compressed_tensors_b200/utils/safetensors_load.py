"""Where each parameter of a safetensors checkpoint lives (utils/safetensors_load.py:84-291 of the reference):
header parsing, name -> file maps for single files, single-file folders and sharded folders with an index, and
the nesting of a layer's compression parameters under the layer's name.  Only metadata is read here; tensors are
opened lazily by the compressors, straight onto the GPU that decompresses them."""
import json
import os
import struct
from typing import Dict, Iterable, Tuple, Union

__all__ = [
    "SAFE_WEIGHTS_NAME", "SAFE_WEIGHTS_INDEX_NAME", "get_safetensors_header", "get_weight_mappings",
    "get_nested_weight_mappings", "get_nested_mappings_from_state_dict", "is_quantization_param",
]

SAFE_WEIGHTS_NAME = "model.safetensors"
SAFE_WEIGHTS_INDEX_NAME = "model.safetensors.index.json"

WeightMappingType = Dict[str, str]
NestedWeightMappingType = Dict[str, WeightMappingType]


def get_safetensors_header(safetensors_path: str) -> Dict[str, object]:
    """The JSON header of a safetensors file: 8 bytes little-endian length, then that many bytes of JSON."""
    with open(safetensors_path, "rb") as f:
        (length,) = struct.unpack("<Q", f.read(8))
        return json.loads(f.read(length).decode("utf-8"))


def get_weight_mappings(path_to_model_or_tensors: str) -> WeightMappingType:
    """{parameter name: path of the file that holds it} for a safetensors file, a folder with one
    `model.safetensors`, or a sharded folder with `model.safetensors.index.json`."""
    path = path_to_model_or_tensors
    if os.path.isfile(path):
        return {k: path for k in get_safetensors_header(path) if k != "__metadata__"}
    single, index = os.path.join(path, SAFE_WEIGHTS_NAME), os.path.join(path, SAFE_WEIGHTS_INDEX_NAME)
    if os.path.exists(single):
        return {k: single for k in get_safetensors_header(single) if k != "__metadata__"}
    if os.path.exists(index):
        with open(index, "r", encoding="utf-8") as f:
            return {k: os.path.join(path, v) for k, v in json.load(f)["weight_map"].items()}
    raise ValueError(f"Could not find a safetensors weight or index file at {path}")


def _split(key: str, params_to_nest: Iterable[str]):
    for p in params_to_nest:
        if key == p or key.endswith("." + p):
            return key[: -len(p)].rstrip("."), p
    return None


def get_nested_weight_mappings(model_path: str, params_to_nest: Iterable[str], return_unmatched_params: bool = False
                               ) -> Union[NestedWeightMappingType, Tuple[NestedWeightMappingType, WeightMappingType]]:
    """{layer: {compression parameter: file}} for every key of the checkpoint that ends in one of
    `params_to_nest`; optionally also the flat map of everything else."""
    params_to_nest = tuple(params_to_nest)
    nested: NestedWeightMappingType = {}
    unmatched: WeightMappingType = {}
    for key, location in get_weight_mappings(model_path).items():
        hit = _split(key, params_to_nest)
        if hit is None:
            unmatched[key] = location
        else:
            nested.setdefault(hit[0], {})[hit[1]] = location
    return (nested, unmatched) if return_unmatched_params else nested


def get_nested_mappings_from_state_dict(state_dict, params_to_nest: Iterable[str], return_unmatched_params: bool = False):
    """The same nesting over an in-memory state dict: {layer: {compression parameter: tensor}}."""
    params_to_nest = tuple(params_to_nest)
    nested, unmatched = {}, {}
    for key, value in state_dict.items():
        hit = _split(key, params_to_nest)
        if hit is None:
            unmatched[key] = value
        else:
            nested.setdefault(hit[0], {})[hit[1]] = value
    return (nested, unmatched) if return_unmatched_params else nested


def is_quantization_param(name: str) -> bool:
    """Whether a parameter name is a scale / zero point / g_idx rather than a weight or bias."""
    return name.endswith(("_scale", "zero_point", "g_idx"))
