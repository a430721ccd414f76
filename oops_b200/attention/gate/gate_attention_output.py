"""``gate_attention_output`` and the gate fused into triangle attention's epilogue.

``gate_attention_output`` keeps the signature, argument meaning and error texts of
``oops/attention/gate/gate_attention_output.py:36-100`` (shape contract ``_contract.py:27-48``,
math ``composed.py:47-53``): ``linear(sigmoid(linear(single, gate_weight)) * attention_flat, output_weight)``.
The two linear maps are plain library GEMMs; the element-wise core between them -- the sigmoid gate on the
attention values, including the move from the head-major ``(*, H, Q, D)`` attention layout to the token-major
``(*, Q, H*D)`` layout of the projection -- is a hand-written kernel behind the C ABI
(``oops_ta_gate_forward`` / ``oops_ta_gate_backward``).

``triangle_attention_gated`` is the fused form this library adds: triangle attention whose forward kernel applies
the gate to its output tile while it is still in registers, so the ``(*, R, C, H*D)`` attention values are never
written and re-read between the two operators at inference, and only written once more (for the reverse pass) in
training.  Dense inputs only; ragged (NestedTensor) operands of the reference's gate operator are not served.
"""

from __future__ import annotations

from typing import Optional

import torch
from torch import Tensor
from torch.nn import functional as F

from ...runtime import cabi, require_no_forward_mode, require_same_device, unsupported
from ...runtime.nested_tensor import is_nested
from ..triangle import function as _function
from ..triangle.triangle_attention import (
    _check_admission, _check_dense_shapes, _flags, _require_bool_mask, _unit_inner,
)

_OPERATOR = "gate_attention_output"


def _check_gate_output(attention: Tensor, single: Tensor, gate_weight: Tensor, output_weight: Tensor) -> None:
    """Shape contract of the reference (oops/attention/gate/_contract.py:27-48), same messages."""
    rank = attention.dim()
    if rank not in (3, 4, 5):
        raise ValueError(
            "attention must have layout (num_heads, query_length, head_size) under optional batch and sample axes"
        )
    if single.dim() + 1 != rank:
        raise ValueError("single must have layout (..., query_length, single_channels)")
    if gate_weight.dim() != 2 or output_weight.dim() != 2:
        raise ValueError("gate_weight and output_weight must be rank-2 matrices")
    lead, (heads, length, head_size) = tuple(attention.shape[:-3]), tuple(attention.shape[-3:])
    channels = heads * head_size
    if tuple(single.shape[:-1]) != (*lead, length):
        raise ValueError("single must share the attention leading axes and its query_length")
    if tuple(gate_weight.shape) != (channels, single.shape[-1]):
        raise ValueError("gate_weight must have shape (num_heads * head_size, single_channels)")
    if output_weight.shape[1] != channels:
        raise ValueError("output_weight input channels must equal num_heads * head_size")


def _pair_view(tensor: Tensor, heads: int, head_size: int, head_major: bool) -> Tensor:
    """View ``(B, H, Q, D)`` (head-major) or ``(B, Q, H*D)`` (token-major) as the C ABI's ``(B, 1, Q, H, D)``."""
    if head_major:
        return tensor.permute(0, 2, 1, 3).unsqueeze(1)
    return tensor.unflatten(-1, (heads, head_size)).unsqueeze(1)


def _run_gate(attention5: Tensor, gate5: Tensor, out5: Tensor) -> None:
    lib = cabi.library()
    batch, rows, cols, heads, head_size = attention5.shape
    a, g, o = cabi.pair_of(attention5), cabi.pair_of(gate5), cabi.pair_of(out5)
    with torch.cuda.device(attention5.device):
        status = lib.oops_ta_gate_forward(
            cabi.DTYPE_CODE[attention5.dtype], batch, rows, cols, heads, head_size, cabi.byref(a), cabi.byref(g), cabi.byref(o),
            torch.cuda.current_stream(attention5.device).cuda_stream,
        )
    if status:
        raise RuntimeError(f"{_OPERATOR} gate kernel failed: {cabi.status_message(status)}")


def _run_gate_backward(attention5: Tensor, gate5: Tensor, dout5: Tensor, dattention5: Optional[Tensor],
                       dgate5: Optional[Tensor]) -> None:
    lib = cabi.library()
    batch, rows, cols, heads, head_size = attention5.shape
    a, g, u = cabi.pair_of(attention5), cabi.pair_of(gate5), cabi.pair_of(dout5)
    da, dg = cabi.pair_of(dattention5), cabi.pair_of(dgate5)
    with torch.cuda.device(attention5.device):
        status = lib.oops_ta_gate_backward(
            cabi.DTYPE_CODE[attention5.dtype], batch, rows, cols, heads, head_size, cabi.byref(a), cabi.byref(g), cabi.byref(u),
            cabi.byref(da), cabi.byref(dg), torch.cuda.current_stream(attention5.device).cuda_stream,
        )
    if status:
        raise RuntimeError(f"{_OPERATOR} gate kernel failed: {cabi.status_message(status)}")


class _SigmoidGate(torch.autograd.Function):
    """``gated[b, q, h*D + d] = sigmoid(gate[b, q, h*D + d]) * attention[b, h, q, d]``."""

    @staticmethod
    def forward(ctx, attention: Tensor, gate: Tensor) -> Tensor:
        batch, heads, length, head_size = attention.shape
        attention, gate = _unit_inner(attention), gate.contiguous()
        gated = torch.empty_like(gate)
        _run_gate(_pair_view(attention, heads, head_size, True), _pair_view(gate, heads, head_size, False),
                  _pair_view(gated, heads, head_size, False))
        ctx.save_for_backward(attention, gate)
        return gated

    @staticmethod
    def backward(ctx, grad_gated: Tensor):
        attention, gate = ctx.saved_tensors
        batch, heads, length, head_size = attention.shape
        attention = _unit_inner(attention)
        grad_gated = grad_gated.resolve_neg().to(gate.dtype).contiguous()
        d_attention = torch.empty(attention.shape, dtype=attention.dtype, device=attention.device) if ctx.needs_input_grad[0] else None
        d_gate = torch.empty_like(gate) if ctx.needs_input_grad[1] else None
        _run_gate_backward(
            _pair_view(attention, heads, head_size, True), _pair_view(gate, heads, head_size, False),
            _pair_view(grad_gated, heads, head_size, False),
            None if d_attention is None else _pair_view(d_attention, heads, head_size, True),
            None if d_gate is None else _pair_view(d_gate, heads, head_size, False),
        )
        return d_attention, d_gate


def gate_attention_output(attention, single, gate_weight: Tensor, output_weight: Tensor):
    r"""Apply a sigmoid gate and output projection to head-major attention values.

    ``linear(sigmoid(linear(single, gate_weight)) * attention_flat, output_weight)`` where ``attention_flat`` puts the
    heads and channels of a query token next to each other.

    Args:
        attention: dense ``(*prefix, H, Q, D)`` values of rank 3, 4 or 5.
        single: gating input ``(*prefix, Q, C)`` on the attention device.
        gate_weight: ``(H * D, C)``; output_weight: ``(O, H * D)``.

    Returns:
        ``(*prefix, Q, O)``.

    Raises:
        ValueError: ranks, shapes, devices or dense/ragged representations disagree.
        OOpsUnsupportedError: ragged operands, non-CUDA tensors, unsupported dtypes.
    """
    if is_nested(attention) or is_nested(single):
        if is_nested(attention) != is_nested(single):
            raise ValueError(
                "gate_attention_output nested attention requires a NestedTensor single"
                if is_nested(attention) else "gate_attention_output dense attention cannot use a NestedTensor single"
            )
        raise unsupported(_OPERATOR, "does not serve NestedTensor operands in this library (dense inputs only)")
    _check_gate_output(attention, single, gate_weight, output_weight)
    require_same_device(_OPERATOR, attention, single, gate_weight, output_weight)
    require_no_forward_mode(_OPERATOR, attention, single, gate_weight, output_weight)
    if not attention.is_cuda or attention.dtype not in cabi.DTYPE_CODE or single.dtype != attention.dtype:
        raise unsupported(
            _OPERATOR, "requires CUDA float16/bfloat16/float32 attention and single of one dtype",
            attention=f"{tuple(attention.shape)} {attention.dtype} {attention.device}", single_dtype=single.dtype,
        )
    lead = tuple(attention.shape[:-3])
    attention4 = attention.reshape(-1, *attention.shape[-3:]) if len(lead) != 1 else attention
    single3 = single.reshape(-1, *single.shape[-2:]) if len(lead) != 1 else single
    gate = F.linear(single3, gate_weight.to(single3.dtype))
    gated = _SigmoidGate.apply(attention4, gate)
    result = F.linear(gated, output_weight.to(gated.dtype))
    return result.reshape(*lead, *result.shape[-2:]) if len(lead) != 1 else result


# ----------------------------------------------------------------------------------------------
# the gate fused into triangle attention
# ----------------------------------------------------------------------------------------------


class _GatedTriangleAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, query, key, value, gate, mask, bias, scale, flags):
        needs_grad = any(ctx.needs_input_grad[i] for i in (0, 1, 2, 3, 5))
        gated, plain, lse = _run_forward_gated(query, key, value, gate, mask, bias, scale, flags, keep_plain=needs_grad)
        ctx.set_materialize_grads(False)
        if needs_grad:
            ctx.save_for_backward(query, key, value, gate, mask, bias, plain, lse)
            ctx.scale, ctx.flags = scale, flags
        return gated

    @staticmethod
    def backward(ctx, grad_gated):
        if grad_gated is None:
            return (None,) * 8
        query, key, value, gate, mask, bias, plain, lse = ctx.saved_tensors
        geometry = _function.DenseGeometry()
        query, key, value, plain, gate = (geometry.canonical_pair(t) for t in (query, key, value, plain, gate))
        grad_gated = geometry.canonical_pair(grad_gated.resolve_neg().to(query.dtype))
        need_q, need_k, need_v, need_g, need_b = (ctx.needs_input_grad[i] for i in (0, 1, 2, 3, 5))
        # through the gate: d(attention) = d(gated) * sigmoid(gate), d(gate) = d(gated) * attention * s (1 - s)
        d_plain = torch.empty_like(plain)
        d_gate = torch.empty_like(gate) if need_g else None
        _run_gate_backward(plain, gate, grad_gated, d_plain, d_gate)
        dq = dk = dv = dbias = None
        if need_q or need_k or need_v or (need_b and bias is not None):
            dq, dk, dv, dbias = _function.run_backward(
                geometry, d_plain, query, key, value, mask, bias, plain, lse.contiguous(), ctx.scale, ctx.flags,
                (need_q, need_k, need_v, need_b),
            )
        return dq, dk, dv, d_gate, None, dbias, None, None


def _run_forward_gated(query, key, value, gate, mask, bias, scale, flags, keep_plain):
    lib = cabi.library()
    device = query.device
    gated = torch.empty(query.shape, dtype=query.dtype, device=device)
    plain = torch.empty(query.shape, dtype=query.dtype, device=device) if keep_plain else None
    batch, rows, cols, heads, _ = query.shape
    lse = torch.empty(batch * rows * heads * cols, dtype=torch.float32, device=device) if keep_plain else None
    with torch.cuda.device(device):
        problem = cabi.make_problem(query, key, value, mask, bias, scale, flags)
        status = lib.oops_ta_supported(cabi.byref(problem))
        if status:
            _function._raise_status(status, "gated forward")
        nbytes = lib.oops_ta_forward_workspace_bytes(cabi.byref(problem))
        scratch = _function._workspace(nbytes, device)
        if scratch is not None:
            problem.workspace, problem.workspace_bytes = scratch.data_ptr(), scratch.numel()
        gate_pair, gated_pair, plain_pair = cabi.pair_of(gate), cabi.pair_of(gated), cabi.pair_of(plain)
        status = lib.oops_ta_forward_gated(
            cabi.byref(problem), cabi.byref(gate_pair), cabi.byref(gated_pair), cabi.byref(plain_pair),
            None if lse is None else lse.data_ptr(), torch.cuda.current_stream(device).cuda_stream,
        )
        if status:
            _function._raise_status(status, "gated forward")
        _function._raise_if_device_failed("gated forward")
    return gated, plain, lse


def triangle_attention_gated(query: Tensor, key: Tensor, value: Tensor, gate: Tensor, mask: Optional[Tensor] = None,
                             triangle_bias: Optional[Tensor] = None, *, scale: Optional[float] = None) -> Tensor:
    r"""``sigmoid(gate) * triangle_attention(query, key, value, mask, triangle_bias, scale=scale)`` in one forward kernel.

    ``gate`` holds the gate logits of the output projection, ``linear(pair, gate_weight)``, with the query's shape
    ``(B, R, C, H, D)`` (or ``(B, R, C, H * D)``); the result has the query's shape and feeds the output projection.
    Dense rank-5 inputs; everything else as ``triangle_attention``.  Gradients flow to query, key, value, gate and bias.
    """
    operator = "triangle_attention_gated"
    for operand in (query, key, value, gate, mask, triangle_bias):
        if operand is not None and is_nested(operand):
            raise unsupported(operator, "serves dense inputs only")
    if query.dim() != 5:
        raise ValueError(f"{operator} query must be (batch, rows, cols, num_heads, head_size), got rank {query.dim()}")
    _check_dense_shapes(query, key, value, mask, triangle_bias)
    if gate.dim() == 4 and gate.shape[-1] == query.shape[-2] * query.shape[-1]:
        gate = gate.unflatten(-1, tuple(query.shape[-2:]))
    if tuple(gate.shape) != tuple(query.shape) or gate.dtype != query.dtype:
        raise ValueError(f"{operator} gate must have the query's shape {tuple(query.shape)} and dtype, got {tuple(gate.shape)} {gate.dtype}")
    require_same_device(operator, query, key, value, gate, mask, triangle_bias)
    require_no_forward_mode(operator, query, key, value, gate, triangle_bias)
    _require_bool_mask(mask)
    _check_admission(query, key, value, mask, triangle_bias,
                     "requires CUDA float16/bfloat16/float32 q/k/v of one dtype and shape with head_size <= 256")
    batch, rows, cols, _heads, head_size = query.shape
    q5 = _function.DenseGeometry().canonical_pair(_unit_inner(query))
    k5 = q5 if key is query else _function.DenseGeometry().canonical_pair(_unit_inner(key))
    v5 = q5 if value is query else k5 if value is key else _function.DenseGeometry().canonical_pair(_unit_inner(value))
    g5 = _unit_inner(gate)
    mask3 = None if mask is None else mask.expand(batch, rows, cols)
    bias5 = None
    if triangle_bias is not None:
        bias5 = triangle_bias.resolve_neg().resolve_conj().contiguous()
        if bias5.element_size() == 2 and cols % 8 != 0:
            bias5 = torch.nn.functional.pad(bias5, (0, -cols % 8))[..., :cols]
    scale = head_size**-0.5 if scale is None else float(scale)
    return _GatedTriangleAttention.apply(q5, k5, v5, g5, mask3, bias5, scale, _flags())


__all__ = ["gate_attention_output", "triangle_attention_gated"]
