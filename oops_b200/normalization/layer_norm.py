"""Layer normalisation over the final feature axis, with the reference's call surface.

Mirrors ``oops/normalization/layer_norm/layer_norm.py:37-154`` of the reference: CUDA float16 / bfloat16 / float32
activations ``(..., C)`` with ``1 <= C <= 8192`` (or a packed ragged batch whose last element axis is static and
physically last), optional ``weight`` / ``bias`` of shape ``(C,)`` in the activation dtype or, for 16-bit activations,
float32.  The kernels are ``oops_ta_layer_norm_forward/_backward`` of the C ABI (``include/oops_ta.h``); there is no
fallback.  Differences from the reference: activations are viewed as ``(rows, C)`` with contiguous rows (other
layouts are copied once, as ``Tensor.reshape`` does); autocast promotion is not re-implemented (parameters must already
be of an accepted dtype); the call is not registered as a ``torch.compile`` custom op.
"""

from __future__ import annotations

import math
from typing import Iterable, Optional

import torch
from torch import Tensor

from ..runtime import cabi, require_no_forward_mode, require_same_device, unsupported
from ..runtime.nested_tensor import is_nested

_NAME = "layer_norm"
_MAX_WIDTH = 8192
_DTYPE_CODES = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}
_HALF = (torch.float16, torch.bfloat16)


def _rows_of(t: Tensor, width: int) -> Tensor:
    """`t` as (rows, width) with contiguous rows; a view when the layout allows it."""
    flat = t.reshape(-1, width)
    if (width > 1 and flat.stride(1) != 1) or (flat.shape[0] > 1 and flat.stride(0) < width):
        flat = flat.contiguous()
    return flat


def _check_status(status: int) -> None:
    if status:
        raise unsupported(_NAME, cabi.status_message(status))


class _LayerNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x: Tensor, weight: Optional[Tensor], bias: Optional[Tensor], eps: float):
        width = x.shape[-1]
        rows_in = _rows_of(x.detach(), width)
        rows = rows_in.shape[0]
        out = torch.empty((rows, width), dtype=x.dtype, device=x.device)
        mean = torch.empty(rows, dtype=torch.float32, device=x.device)
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        affine = next((p for p in (weight, bias) if p is not None), None)
        affine_code = _DTYPE_CODES[affine.dtype if affine is not None else x.dtype]
        w = weight.detach().contiguous() if weight is not None else None
        b = bias.detach().contiguous() if bias is not None else None
        lib = cabi.library()
        with torch.cuda.device(x.device):
            _check_status(lib.oops_ta_layer_norm_forward(
                _DTYPE_CODES[x.dtype], affine_code, rows, width, rows_in.data_ptr(), rows_in.stride(0) if rows > 1 else width,
                w.data_ptr() if w is not None else None, b.data_ptr() if b is not None else None, float(eps), out.data_ptr(), width,
                mean.data_ptr(), rstd.data_ptr(), torch.cuda.current_stream(x.device).cuda_stream))
        ctx.save_for_backward(rows_in, w if w is not None else torch.empty(0), mean, rstd)
        ctx.has_weight, ctx.has_bias = weight is not None, bias is not None
        ctx.affine_code, ctx.affine_dtype = affine_code, (affine.dtype if affine is not None else x.dtype)
        ctx.shape = x.shape
        return out.view(x.shape)

    @staticmethod
    def backward(ctx, grad_out: Tensor):
        rows_in, w, mean, rstd = ctx.saved_tensors
        rows, width = rows_in.shape
        dy = _rows_of(grad_out, width)
        need_x, need_w, need_b = ctx.needs_input_grad[0], ctx.has_weight and ctx.needs_input_grad[1], ctx.has_bias and ctx.needs_input_grad[2]
        device = rows_in.device
        dx = torch.empty((rows, width), dtype=rows_in.dtype, device=device) if need_x else None
        dw = torch.zeros(width, dtype=ctx.affine_dtype, device=device) if need_w else None
        db = torch.zeros(width, dtype=ctx.affine_dtype, device=device) if need_b else None
        lib = cabi.library()
        if rows > 0:
            need = lib.oops_ta_layer_norm_backward_workspace_bytes(rows, width) if (need_w or need_b) else 0
            scratch = torch.empty(max(int(need), 1), dtype=torch.uint8, device=device)
            with torch.cuda.device(device):
                _check_status(lib.oops_ta_layer_norm_backward(
                    _DTYPE_CODES[rows_in.dtype], ctx.affine_code, rows, width, dy.data_ptr(), dy.stride(0) if rows > 1 else width,
                    rows_in.data_ptr(), rows_in.stride(0) if rows > 1 else width, w.data_ptr() if ctx.has_weight else None,
                    mean.data_ptr(), rstd.data_ptr(), dx.data_ptr() if need_x else None, width,
                    dw.data_ptr() if need_w else None, db.data_ptr() if need_b else None, scratch.data_ptr(), int(need),
                    torch.cuda.current_stream(device).cuda_stream))
        return (dx.view(ctx.shape) if need_x else None), dw, db, None


def layer_norm(input, normalized_shape, weight: Optional[Tensor] = None, bias: Optional[Tensor] = None, eps: float = 1e-5):
    """Normalize the final feature dimension of CUDA activations; see the module docstring."""
    if is_nested(input):
        return _layer_norm_nested(input, normalized_shape, weight, bias, eps)
    require_no_forward_mode(_NAME, input, weight, bias)
    require_same_device(_NAME, input, weight, bias)
    shape = (normalized_shape,) if isinstance(normalized_shape, int) else tuple(normalized_shape)
    if len(shape) != 1:
        raise unsupported(_NAME, "normalizes over the final dimension only", normalized_shape=shape, input_shape=tuple(input.shape))
    width = math.prod(shape)
    affine = [p for p in (weight, bias) if p is not None]
    mixed = input.dtype in _HALF and any(p.dtype is torch.float32 for p in affine) and any(p.dtype is not torch.float32 for p in affine)
    supported = (
        input.is_cuda and input.dim() >= 1 and input.shape[-1] == width and 0 < width <= _MAX_WIDTH and input.dtype in _DTYPE_CODES
        and not mixed
        and all(p.shape == (width,) and (p.dtype is input.dtype or (input.dtype in _HALF and p.dtype is torch.float32)) for p in affine)
    )
    if not supported:
        raise unsupported(_NAME, "requires a CUDA half/float32 activation with a matching contiguous affine row",
                          input_dtype=input.dtype, device=input.device, normalized_size=width,
                          weight_dtype=None if weight is None else weight.dtype, bias_dtype=None if bias is None else bias.dtype)
    if input.numel() == 0:
        raise unsupported(_NAME, "does not serve an empty input", input_shape=tuple(input.shape))
    return _LayerNorm.apply(input, weight, bias, eps)


def _layer_norm_nested(input, normalized_shape, weight, bias, eps):
    if is_nested(weight) or is_nested(bias):
        raise ValueError(f"{_NAME} NestedTensor input requires dense affine parameters")
    if input.dim() < 2 or not input.ragged_dims:
        raise unsupported(_NAME, "requires a NestedTensor with explicit packed element topology", ragged_dims=input.ragged_dims)
    normalized_dim = input.dim() - 2
    if normalized_dim in input.ragged_dims or input.packed_dim_order[-1] != normalized_dim:
        raise unsupported(_NAME, "requires the final logical element dimension to be static and physically last",
                          ragged_dims=input.ragged_dims, packed_dim_order=input.packed_dim_order)
    packed = input.concat
    if packed.dim() < 1:
        raise unsupported(_NAME, "requires packed values with a retained static final dimension")
    shape: Iterable[int] = (normalized_shape,) if isinstance(normalized_shape, int) else tuple(normalized_shape)
    return input.packed_like(layer_norm(packed, shape, weight, bias, eps))
