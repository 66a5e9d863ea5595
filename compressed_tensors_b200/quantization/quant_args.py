"""Quantization argument schema (quantization/quant_args.py:30-408 of the reference): same field
names, defaults, validation outcomes and error types, so configs written for the reference load
unchanged.  Only the rounding helper touches the device."""
import warnings
from enum import Enum
from typing import Any, Dict, List, Optional, Union

import torch
from pydantic import BaseModel, ConfigDict, Field, field_validator, model_validator

__all__ = [
    "FP8_DTYPE", "FP8_E4M3_DATA", "FP4_E2M1_DATA", "BFLOAT16_DATA", "FloatArgs", "QuantizationType",
    "QuantizationStrategy", "QuantizationArgs", "round_to_quantized_type", "ActivationOrdering", "DynamicType",
]

FP8_DTYPE = torch.float8_e4m3fn


class FloatArgs:
    exponent: int
    mantissa: int
    bits: Optional[int] = None
    max: Optional[float] = None
    min: Optional[float] = None
    dtype: Optional[torch.dtype] = None


class FP4_E2M1_DATA(FloatArgs):
    exponent, mantissa, bits = 2, 1, 4
    max, min = 6.0, -6.0

    @staticmethod
    def cast_to_fp4(x: torch.Tensor) -> torch.Tensor:
        """Snap to the e2m1 grid with ties to the even code, keeping the dtype
        (quant_args.py:55-68).  Runs as a fake-quantize with unit scale on the device."""
        from .. import torch_ops as ops

        flat = x.reshape(1, -1) if x.ndim != 2 else x
        pad = (-flat.shape[-1]) % 16
        one = torch.ones(1, dtype=torch.float32, device=x.device)
        if pad:
            flat = torch.nn.functional.pad(flat, (0, pad))
        out = ops.quantize(flat, one, None, qtype=ops.QFLOAT, bits=4, col_group=flat.shape[-1], scale_row_stride=0,
                           out_dtype=x.dtype, global_scale=one)
        if pad:
            out = out[..., : flat.shape[-1] - pad]
        return out.reshape(x.shape)


class FP8_E4M3_DATA(FloatArgs):
    exponent, mantissa, bits = 4, 3, 8
    max = torch.finfo(torch.float8_e4m3fn).max
    min = torch.finfo(torch.float8_e4m3fn).min
    dtype = torch.float8_e4m3fn


class BFLOAT16_DATA(FloatArgs):
    exponent, mantissa = 8, 7


class QuantizationType(str, Enum):
    INT = "int"
    FLOAT = "float"


class QuantizationStrategy(str, Enum):
    TENSOR = "tensor"
    CHANNEL = "channel"
    GROUP = "group"
    BLOCK = "block"
    TOKEN = "token"
    TENSOR_GROUP = "tensor_group"
    ATTN_HEAD = "attn_head"


class DynamicType(str, Enum):
    LOCAL = "local"


class ActivationOrdering(str, Enum):
    GROUP = "group"
    WEIGHT = "weight"
    DYNAMIC = "dynamic"
    STATIC = "static"

    @staticmethod
    def get_aliases() -> Dict[str, str]:
        return {"dynamic": "group", "static": "weight"}

    def __eq__(self, other):
        if isinstance(other, str):
            a = self.get_aliases()
            mine, theirs = a.get(self.value, self.value), a.get(getattr(other, "value", other), getattr(other, "value", other))
            return mine == theirs
        return NotImplemented

    def __hash__(self):
        return hash(self.get_aliases().get(self.value, self.value))


_DYNAMIC_OK = (QuantizationStrategy.TOKEN, QuantizationStrategy.TENSOR, QuantizationStrategy.TENSOR_GROUP, QuantizationStrategy.GROUP)


class QuantizationArgs(BaseModel, use_enum_values=True):
    num_bits: int = 8
    type: QuantizationType = QuantizationType.INT
    symmetric: bool = True
    group_size: Optional[int] = None
    strategy: Optional[QuantizationStrategy] = None
    block_structure: Optional[List[int]] = None
    dynamic: Union[DynamicType, bool] = False
    actorder: Union[ActivationOrdering, bool, None] = None
    observer: Optional[str] = Field(default=None)
    observer_kwargs: Dict[str, Any] = Field(default_factory=dict)

    model_config = ConfigDict(extra="forbid")

    @field_validator("type", mode="before")
    def _type(cls, v):
        return QuantizationType(v.lower()) if isinstance(v, str) else v

    @field_validator("group_size", mode="before")
    def _group(cls, v):
        if v is not None and v < -1:
            raise ValueError(f"Invalid group size {v}. Use group_size > 0 for strategy='group' and group_size = -1 for 'channel'")
        return v

    @field_validator("block_structure", mode="before")
    def _block(cls, v):
        if v is None:
            return v
        err = f"Invalid block_structure '{v}'. Must be a list of ints [rows, cols]."
        if isinstance(v, str):
            try:
                return [int(p) for p in v.split("x")]
            except Exception:
                raise ValueError(err)
        if isinstance(v, (list, tuple)) and len(v) == 2 and all(isinstance(p, int) for p in v):
            return list(v)
        raise ValueError(err)

    @field_validator("strategy", mode="before")
    def _strategy(cls, v):
        return QuantizationStrategy(v.lower()) if isinstance(v, str) else v

    @field_validator("actorder", mode="before")
    def _actorder(cls, v):
        if isinstance(v, bool):
            return ActivationOrdering.GROUP if v else None
        if isinstance(v, str):
            return ActivationOrdering(v.lower())
        return v

    @field_validator("dynamic", mode="before")
    def _dynamic(cls, v):
        return DynamicType(v.lower()) if isinstance(v, str) else v

    @model_validator(mode="after")
    def _after(self):
        strategy, g = self.strategy, self.group_size
        if strategy is None:
            if g is None:
                strategy = QuantizationStrategy.TENSOR
            elif g > 0:
                strategy = QuantizationStrategy.GROUP
            elif g == -1:
                strategy = QuantizationStrategy.CHANNEL
            else:
                raise ValueError(f"Invalid group size {g}. Use group_size > 0 for strategy='group' and group_size = -1 for 'channel'")
        strategy = QuantizationStrategy(strategy)
        if strategy == QuantizationStrategy.TOKEN and not self.dynamic:
            raise ValueError("Cannot perform static token quantization, please use `dynamic=True`")
        grouped = strategy in (QuantizationStrategy.GROUP, QuantizationStrategy.TENSOR_GROUP)
        if grouped and (g is None or g <= 0):
            raise ValueError(f"strategy {strategy} requires group_size to be set to a positive value")
        if g is not None and g > 0 and not grouped:
            raise ValueError("group_size requires strategy to be set to 'group'")
        if (strategy == QuantizationStrategy.BLOCK) != (self.block_structure is not None):
            raise ValueError("Block strategy requires block structure" if strategy == QuantizationStrategy.BLOCK
                             else "Block structure requires block strategy")
        if self.actorder is not None and strategy != QuantizationStrategy.GROUP:
            raise ValueError("Must use group quantization strategy in order to apply activation ordering")
        observer = self.observer
        if self.dynamic:
            if strategy not in _DYNAMIC_OK:
                raise ValueError(f"One of {_DYNAMIC_OK} must be used for dynamic quant.")
            if self.dynamic == DynamicType.LOCAL and strategy != QuantizationStrategy.TENSOR_GROUP:
                raise ValueError("local is only supported for strategy tensor_group")
            if observer is not None:
                if self.dynamic is True:
                    if observer != "memoryless":
                        warnings.warn("No observer is used for dynamic quant., setting to None")
                    observer = None
            elif self.dynamic == DynamicType.LOCAL:
                observer = "minmax"
        elif observer is None:
            observer = "minmax"
        self.strategy = strategy.value
        self.observer = observer
        return self

    def pytorch_dtype(self) -> torch.dtype:
        if self.type == QuantizationType.FLOAT:
            if self.num_bits == 8:
                return FP8_E4M3_DATA.dtype
            raise NotImplementedError("Only num_bits in (8) are supported")
        if self.type == QuantizationType.INT:
            return torch.int8 if self.num_bits <= 8 else (torch.int16 if self.num_bits <= 16 else torch.int32)
        raise ValueError(f"Invalid quantization type {self.type}")

    def get_observer(self) -> Optional[str]:
        return self.observer


def round_to_quantized_type(tensor: torch.Tensor, args: QuantizationArgs) -> torch.Tensor:
    """Round to the nearest value of the quantized type, keeping the dtype (quant_args.py:384-408)."""
    from .. import torch_ops as ops

    if args.type == QuantizationType.FLOAT:
        if args.num_bits == 4:
            return FP4_E2M1_DATA.cast_to_fp4(tensor)
        if args.num_bits != 8:
            raise NotImplementedError("Only num_bits in (4, 8) are supported")
        qtype, bits = ops.QFLOAT, 8
    elif args.type == QuantizationType.INT:
        qtype, bits = ops.QINT, 8
    else:
        raise ValueError(f"Invalid quantization type {args.type}")
    flat = tensor.reshape(1, -1)
    one = torch.ones(1, dtype=tensor.dtype, device=tensor.device)
    if qtype == ops.QINT:
        # torch.round without clamping: run the int path through a range that cannot clip (8-bit is the widest built),
        # so large magnitudes go through a float32 detour instead
        return torch.round(tensor)
    out = ops.quantize(flat, one, None, qtype=qtype, bits=bits, col_group=flat.shape[-1], scale_row_stride=0, out_dtype=tensor.dtype)
    return out.reshape(tensor.shape)
