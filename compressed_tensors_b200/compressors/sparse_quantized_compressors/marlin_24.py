"""Marlin24Compressor (compressors/sparse_quantized_compressors/marlin_24.py of the reference): quantized weights
with a 2:4 sparsity structure in the layout of the Marlin-24 kernel.  Every step of the per-weight pipeline runs
on the GPU: quantize to int codes, check the 2:4 structure, CUTLASS 2:4 compaction + reordered metadata, tile
permutation + packing of the codes, permutation of the scales.  As in the reference, decompression is not
implemented for this format."""
from typing import Dict, Generator, Tuple

import torch
from torch import Tensor

from ... import torch_ops as ops
from ..._lib import on_gpu
from ...config import CompressionFormat
from ...quantization.lifecycle.forward import quantize
from ...quantization.quant_args import QuantizationArgs, QuantizationStrategy
from ...utils.helpers import merge_names
from ...utils.safetensors_load import is_quantization_param
from ..base import BaseCompressor

__all__ = ["Marlin24Compressor", "compress_weight_24", "pack_weight_24", "pack_scales_24", "tensor_follows_mask_structure"]


def tensor_follows_mask_structure(tensor: Tensor, mask: str = "2:4") -> bool:
    """utils/helpers.py:93-115: at least n zeros in every chunk of m consecutive elements; raises ValueError if not."""
    n, m = (int(v) for v in mask.split(":"))
    zero_counts = (tensor.reshape(-1, m) == 0).sum(dim=1)
    if not bool(torch.all(zero_counts >= n)):
        raise ValueError()
    return True


def compress_weight_24(weight: Tensor) -> Tuple[Tensor, Tensor]:
    """marlin_24.py:202-206: CUTLASS 2:4 compaction -> (values [rows, cols/2], reordered int16 meta [rows, cols/16])."""
    return ops.cutlass24_compress(on_gpu(weight).contiguous())


def pack_weight_24(weight: Tensor, quantization_args: QuantizationArgs, tile: int = 16) -> Tensor:
    """marlin_24.py:225-249 on the reference's operand: unsigned codes [size_k, size_n] (input dimension first).
    The kernel takes the codes before the transpose and the shift, so both are undone here."""
    if tile != 16:
        raise NotImplementedError("Marlin-24 tiles are 16 x 64")
    half = (1 << quantization_args.num_bits) // 2
    codes = (on_gpu(weight).t().to(torch.int32) - half).to(torch.int8).contiguous()
    return ops.marlin24_pack_weight(codes, quantization_args.num_bits)


def pack_scales_24(scales: Tensor, quantization_args: QuantizationArgs, w_shape: torch.Size) -> Tensor:
    """marlin_24.py:252-273 on the reference's operand: scales [groups, size_n] (already transposed)."""
    grouped = quantization_args.strategy == QuantizationStrategy.GROUP.value and quantization_args.group_size < w_shape[0]
    return ops.marlin24_pack_scales(on_gpu(scales).t().contiguous(), grouped)


@BaseCompressor.register(name=CompressionFormat.marlin_24.value)
class Marlin24Compressor(BaseCompressor):
    @staticmethod
    def validate_quant_compatability(names_to_scheme) -> bool:
        """marlin_24.py:44-89: weight schemes only, group (128) or channel strategy, symmetric."""
        for name, scheme in names_to_scheme.items():
            args = scheme.weights
            if args is None:
                raise ValueError("Marlin24 Compressor is only valid for weight quantization schemes")
            if args.strategy not in (QuantizationStrategy.GROUP.value, QuantizationStrategy.CHANNEL.value):
                raise ValueError(f"Marlin24 Compressor is only valid for group and channel quantization strategies, got {args.strategy} in {name}")
            if args.group_size is not None and args.group_size != 128:
                raise ValueError(f"Marlin24 Compressor is only valid for group size 128, got {args.group_size} in {name}")
            if not args.symmetric:
                raise ValueError(f"Marlin24 Compressor is only valid for symmetric quantzation, got symmetric={args.symmetric} in {name}")
        return True

    @staticmethod
    def validate_sparsity_structure(name: str, weight: Tensor) -> bool:
        """marlin_24.py:91-113."""
        try:
            return tensor_follows_mask_structure(weight)
        except ValueError:
            raise ValueError("Marlin24 Compressor is only compatible with weights that have a 2:4 sparsity structure. "
                             f"Found segments in {name} that do not match the expected structure.") from None

    @property
    def compression_param_names(self) -> Tuple[str]:
        return ("weight_packed", "scale_packed", "meta")

    def compress(self, model_state: Dict[str, Tensor], names_to_scheme, show_progress: bool = False, **kwargs) -> Dict[str, Tensor]:
        """marlin_24.py:124-200.  Results are left on the CPU, as the reference leaves them."""
        self.validate_quant_compatability(names_to_scheme)
        out: Dict[str, Tensor] = {}
        for name, value in model_state.items():
            if name.endswith(".weight"):
                prefix = name[: -len(".weight")]
                scale = model_state.get(merge_names(prefix, "weight_scale"))
                if scale is not None:
                    zp = model_state.get(merge_names(prefix, "weight_zero_point"))
                    args = names_to_scheme[prefix].weights
                    scale16 = on_gpu(scale).to(torch.float16)  # the Marlin-24 kernel takes float16
                    codes = quantize(x=on_gpu(value).to(torch.float16), scale=scale16, zero_point=on_gpu(zp), args=args, dtype=torch.int8)
                    self.validate_sparsity_structure(prefix, codes)
                    sparse, meta = ops.cutlass24_compress(codes)
                    size_k = sparse.shape[1]  # the packed weight is input-dimension first: [size_k, size_n]
                    grouped = args.strategy == QuantizationStrategy.GROUP.value and args.group_size < size_k
                    out[merge_names(prefix, "scale_packed")] = ops.marlin24_pack_scales(scale16.contiguous(), grouped).cpu()
                    out[merge_names(prefix, "weight_packed")] = ops.marlin24_pack_weight(sparse, args.num_bits).cpu()
                    out[merge_names(prefix, "meta")] = meta.cpu().reshape(meta.shape[1] // 2, meta.shape[0] * 2)
                    continue
            if not is_quantization_param(name):
                out[name] = value.to("cpu")
        return out

    def decompress(self, path_to_model_or_tensors: str, device: str = "cpu", **kwargs) -> Generator[Tuple[str, Tensor], None, None]:
        raise NotImplementedError("Decompression is not implemented for the Marlin24 Compressor.")
