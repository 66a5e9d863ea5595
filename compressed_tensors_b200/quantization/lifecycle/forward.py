"""quantize / dequantize / fake_quantize with the reference's signatures
(quantization/lifecycle/forward.py:45-189).  The host part only works out how the scale tensor
lines up with the input (strategy -> group geometry) and which dtype the reference would return;
all arithmetic runs in the ctb200 kernels."""
from typing import Optional, Tuple

import torch

from ... import torch_ops as ops
from ..quant_args import QuantizationArgs, QuantizationStrategy
from ..utils.helpers import qtype_code

__all__ = ["quantize", "dequantize", "fake_quantize", "infer_dequant_args", "forward_quantize", "wrap_module_forward_quantized"]

_FLOATS = (torch.bfloat16, torch.float16, torch.float32)


def _promote(a: torch.dtype, b: torch.dtype) -> torch.dtype:
    return a if a == b else torch.float32


def _geometry(x: torch.Tensor, scale: torch.Tensor, args: QuantizationArgs) -> Tuple[int, int, int]:
    """(col_group, row_group, scale_row_stride) for x viewed as [rows, cols]."""
    cols = x.shape[-1]
    rows = x.numel() // cols if cols else 0
    strategy = args.strategy
    if strategy == QuantizationStrategy.BLOCK:
        if x.ndim != 2:
            raise NotImplementedError("block quantization is built for 2-D tensors")
        bh, bw = args.block_structure
        if rows % bh != 0:  # forward.py:215-219
            raise ValueError(f"Tensor height {rows} is not divisible by block_height {bh}. Block quantization requires exact division.")
        if cols % bw != 0:  # forward.py:220-224
            raise ValueError(f"Tensor width {cols} is not divisible by block_width {bw}. Block quantization requires exact division.")
        return bw, bh, cols // bw
    if strategy in (QuantizationStrategy.GROUP, QuantizationStrategy.TENSOR_GROUP):
        g = args.group_size
        if cols >= g and cols % g != 0:  # forward.py:277-282
            raise ValueError(f"tensor column shape must be divisble by the given group_size {g} but got {cols}")
        if cols < g:
            raise ValueError(f"group_size {g} exceeds the {cols} columns of the tensor")
        groups = cols // g
        if scale.numel() == rows * groups:
            return g, 1, groups
        if scale.numel() == groups:  # one row of scales shared by every row
            return g, 1, 0
        raise ValueError(f"scale of shape {tuple(scale.shape)} does not match {rows} rows x {groups} groups")
    # TENSOR / CHANNEL / TOKEN: the scale broadcasts against x
    if scale.numel() == 1:
        return cols, 1, 0
    if scale.numel() == rows and (scale.ndim == 0 or scale.shape[-1] == 1):
        return cols, 1, 1
    raise NotImplementedError(f"strategy {strategy} with a scale of shape {tuple(scale.shape)} against input {tuple(x.shape)} is not built")


def infer_dequant_args(x_q: torch.Tensor, scale: torch.Tensor) -> QuantizationArgs:
    """Strategy inference of dequantize() when args is None (forward.py:106-138)."""
    if scale.ndim in (0, 1):
        return QuantizationArgs(strategy=QuantizationStrategy.TENSOR)
    if scale.ndim == 2:
        if scale.shape[1] == 1:
            return QuantizationArgs(strategy=QuantizationStrategy.CHANNEL)
        if scale.shape[0] == 1 or scale.shape[0] == x_q.shape[0]:
            return QuantizationArgs(strategy=QuantizationStrategy.GROUP, group_size=int(x_q.shape[1] / scale.shape[1]))
        rows, cols = x_q.shape[-2], x_q.shape[-1]
        return QuantizationArgs(strategy=QuantizationStrategy.BLOCK, block_structure=[rows // scale.shape[0], cols // scale.shape[1]])
    raise ValueError(f"Could not infer a quantization strategy from scale with {scale.ndim} dimmensions. Expected 0 or 2 dimmensions.")


_G_IDX_UNSET = {}  # (data_ptr, version, numel) of a g_idx tensor -> whether it holds a -1 (one read-back per tensor state)


def _resolve_g_idx(g_idx: torch.Tensor, col_group: int, cols: int):
    """forward.py:286 `is_column_order = g_idx is None or -1 in g_idx`: a column map that still holds a -1 (the
    value it is initialised with) is ignored.  The answer needs the tensor's contents, so it is read back once per
    tensor state and remembered; while a CUDA graph is being captured nothing may be read back, and the choice is
    made on the device instead (the map or the plain column order, selected by a 0-dim flag)."""
    if g_idx.is_cuda and torch.cuda.is_current_stream_capturing():
        plain = torch.arange(cols, device=g_idx.device, dtype=g_idx.dtype) // col_group
        return torch.where((g_idx == -1).any(), plain, g_idx)
    key = (g_idx.data_ptr(), g_idx._version, g_idx.numel(), g_idx.device)
    unset = _G_IDX_UNSET.get(key)
    if unset is None:
        if len(_G_IDX_UNSET) > 4096:
            _G_IDX_UNSET.clear()
        unset = _G_IDX_UNSET[key] = bool((g_idx == -1).any())
    return None if unset else g_idx


def _common(x, scale, args, g_idx, global_scale):
    if x.dtype not in _FLOATS + (torch.int8, torch.float8_e4m3fn):
        raise TypeError(f"unsupported input dtype {x.dtype}")
    col_group, row_group, srs = _geometry(x, scale, args)
    grouped = args.strategy in (QuantizationStrategy.GROUP, QuantizationStrategy.TENSOR_GROUP)
    use_gidx = _resolve_g_idx(g_idx, col_group, x.shape[-1]) if grouped and g_idx is not None else None
    kw = dict(qtype=qtype_code(args), bits=args.num_bits, col_group=col_group, row_group=row_group, scale_row_stride=srs,
              g_idx=use_gidx, global_scale=global_scale)
    sdt = torch.float32 if global_scale is not None else scale.dtype
    return kw, grouped, sdt


@torch.no_grad()
def quantize(x: torch.Tensor, scale: torch.Tensor, zero_point: Optional[torch.Tensor], args: QuantizationArgs,
             dtype: Optional[torch.dtype] = None, g_idx: Optional[torch.Tensor] = None,
             global_scale: Optional[torch.Tensor] = None) -> torch.Tensor:
    """forward.py:45-81.  Result dtype: `dtype` if given, else the input dtype for GROUP / TENSOR_GROUP
    and the promoted (input, scale) dtype for the other strategies, as in the reference."""
    kw, grouped, sdt = _common(x, scale, args, g_idx, global_scale)
    out_dtype = dtype if dtype is not None else (x.dtype if grouped else _promote(x.dtype, sdt))
    return ops.quantize(x, scale, zero_point, out_dtype=out_dtype, **kw)


@torch.no_grad()
def dequantize(x_q: torch.Tensor, scale: torch.Tensor, zero_point: Optional[torch.Tensor] = None,
               args: Optional[QuantizationArgs] = None, dtype: Optional[torch.dtype] = None,
               g_idx: Optional[torch.Tensor] = None, global_scale: Optional[torch.Tensor] = None) -> torch.Tensor:
    """forward.py:85-153.  `dtype` defaults to the scale dtype and, as in the reference, only the
    GROUP / TENSOR_GROUP path applies it; the other strategies return the scale's compute dtype."""
    if args is None:
        args = infer_dequant_args(x_q, scale)
    if dtype is None:
        dtype = scale.dtype
    kw, grouped, sdt = _common(x_q, scale, args, g_idx, global_scale)
    out_dtype = dtype if grouped else sdt
    if out_dtype not in _FLOATS:
        raise TypeError(f"dequantize cannot produce {out_dtype}")
    return ops.dequantize(x_q, scale, zero_point, out_dtype=out_dtype, **kw)


@torch.no_grad()
def fake_quantize(x: torch.Tensor, scale: torch.Tensor, zero_point: Optional[torch.Tensor], args: QuantizationArgs,
                  g_idx: Optional[torch.Tensor] = None, global_scale: Optional[torch.Tensor] = None) -> torch.Tensor:
    """forward.py:157-189: quantize then dequantize in one kernel."""
    kw, grouped, sdt = _common(x, scale, args, g_idx, global_scale)
    out_dtype = x.dtype if grouped else sdt
    return ops.fake_quantize(x, scale, zero_point, out_dtype=out_dtype, **kw)


@torch.no_grad()
def forward_quantize(module: torch.nn.Module, value: torch.Tensor, base_name: str, args: QuantizationArgs) -> torch.Tensor:
    """forward.py:415-452: fake-quantize `value` ("input", "weight" or "output" of `module`) with the module's static
    qparams, or with qparams computed from the value itself when `args.dynamic` (per token / tensor / group; NVFP4
    activations keep their static `<base_name>_global_scale` and only the local scales are dynamic)."""
    from ..quant_args import DynamicType
    from ..quant_config import QuantizationStatus
    from ..utils.helpers import compute_dynamic_scales_and_zp

    if base_name == "weight" and getattr(module, "quantization_status", None) == QuantizationStatus.COMPRESSED:
        return value  # the stored weight already is the quantized one
    if value.numel() == 0:
        return value
    g_idx = getattr(module, "weight_g_idx", None)
    global_scale = getattr(module, f"{base_name}_global_scale", None)
    group = _fused_dynamic_group(value, args, g_idx, global_scale)
    if group:
        # calibrate + fake-quantize a token / group in one pass: the same bits as the three separate kernels below
        flat = value.reshape(-1, value.shape[-1])
        fake, _ = ops.absmax_quantize(flat, qtype=qtype_code(args), bits=args.num_bits, col_group=group, codec="dtype", out_dtype=torch.bfloat16)
        return fake.reshape(value.shape)
    if args.dynamic in (True, DynamicType.LOCAL):
        scale, zero_point = compute_dynamic_scales_and_zp(value=value, args=args, module=module, global_scale=global_scale)
    else:
        scale = getattr(module, f"{base_name}_scale")
        zero_point = getattr(module, f"{base_name}_zero_point", None)
    return fake_quantize(x=value, scale=scale, zero_point=zero_point, args=args, g_idx=g_idx, global_scale=global_scale)


def _fused_dynamic_group(value: torch.Tensor, args: QuantizationArgs, g_idx, global_scale) -> int:
    """Group size for the single-pass calibrate + fake-quantize kernel, or 0 when the case is not one it is built for:
    dynamic symmetric int (<= 8 bit) / fp8 quantization of a contiguous bf16 tensor, per token ([batch, tokens, hidden]
    with hidden <= 8192) or per power-of-two group of 8..256 elements."""
    cols = value.shape[-1]
    if not (args.dynamic is True and args.symmetric and value.dtype == torch.bfloat16 and value.is_cuda and value.is_contiguous()
            and cols % 8 == 0 and g_idx is None and global_scale is None):
        return 0
    if not (args.num_bits == 8 or (args.type == "int" and args.num_bits < 8)):
        return 0
    if args.strategy == QuantizationStrategy.TOKEN and value.ndim == 3 and cols <= 8192:
        return cols
    if args.strategy == QuantizationStrategy.GROUP and value.ndim >= 2:
        g = args.group_size
        if g and 8 <= g <= 256 and g & (g - 1) == 0 and cols % g == 0:
            return g
    return 0


def wrap_module_forward_quantized(module: torch.nn.Module, scheme) -> None:
    """forward.py:355-412: replace `module.forward` by a forward that fake-quantizes the input activations, runs the
    layer on a fake-quantized copy of the weight (restored afterwards) and fake-quantizes the output, each only where
    the scheme asks for it; `module.quantization_enabled = False` bypasses all of it.  The module must carry the
    parameters that initialize_module_for_quantization registers."""
    import functools

    from ..quant_config import QuantizationStatus

    plain = module.forward  # bound method (or partial) of the un-wrapped layer

    @functools.wraps(getattr(plain, "__func__", plain))
    def quantized_forward(self, *args, **kwargs):
        if not getattr(self, "quantization_enabled", True):
            return plain(*args, **kwargs)
        x = args[0]
        status = getattr(self, "quantization_status", None)
        fake_weight = scheme.weights is not None and status != QuantizationStatus.COMPRESSED
        if scheme.input_activations is not None:
            x = forward_quantize(self, x, "input", scheme.input_activations)
        if fake_weight:
            kept = self.weight.data
            self.weight.data = forward_quantize(self, self.weight.data, "weight", scheme.weights)
        try:
            out = plain(x, *args[1:], **kwargs)
        finally:
            if fake_weight:
                self.weight.data = kept
        if scheme.output_activations is not None:
            calibrating_static = status == QuantizationStatus.CALIBRATION and not scheme.output_activations.dynamic
            if not calibrating_static:  # static output qparams are still being observed: leave the output alone
                out = forward_quantize(self, out, "output", scheme.output_activations)
        return out

    module.forward = quantized_forward.__get__(module, module.__class__)
