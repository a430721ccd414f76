"""Autograd boundary of triangle attention over the C ABI.

Takes the place of ``oops/attention/triangle/triton/ops.py`` in the reference
(``_TriangleAttention`` :413, ``_setup_context`` :369, ``_backward_from_context``
:380): gradients for query, key, value and bias only; mask and the saved
log-sum-exp are not differentiable; undefined upstream gradients are not
materialised; the reverse pass honours ``needs_input_grad`` subsets; no double
backward.

A call is described by a *geometry*: a recipe that turns the tensors handed to
the Function into one or more uniform ``(B, R, C, H, D)`` views, each of which is
one C-ABI problem.  Dense inputs are a single view (the tensor itself, whatever
its strides).  A packed ragged batch is one view per sample, computed from the
packed layout the reference documents in ``oops/attention/triangle/nested.py:
275-288`` (cell start, cell stride = number of prefixes, bias start/strides).
"""

from __future__ import annotations

from contextlib import contextmanager
from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import torch
from torch import Tensor

from ...runtime import cabi


@dataclass(frozen=True)
class DenseGeometry:
    """One uniform problem: the tensors are already ``(B, R, C, H, D)`` views."""

    def pair_views(self, tensor: Tensor) -> List[Tensor]:
        return [tensor]

    def mask_views(self, mask: Tensor) -> List[Tensor]:
        return [mask]

    def bias_views(self, bias: Tensor) -> List[Tensor]:
        return [bias]

    def lse_sizes(self, query: Tensor) -> List[Tuple[int, int, int, int]]:
        batch, rows, cols, heads, _ = query.shape
        return [(batch, rows, heads, cols)]

    def canonical_pair(self, tensor: Tensor) -> Tensor:
        """Unit inner stride; 16-bit tensors additionally get 16-byte aligned rows, which the TMA kernels need."""
        if tensor.shape[-1] != 1 and tensor.stride(-1) != 1:
            return tensor.contiguous()
        if tensor.element_size() == 2 and (
            tensor.data_ptr() % 16 != 0
            or any(size > 1 and (stride <= 0 or stride % 8 != 0) for size, stride in zip(tensor.shape[:-1], tensor.stride()[:-1]))
        ):
            return tensor.contiguous()
        return tensor

    def canonical_bias(self, bias: Tensor) -> Tensor:
        return bias


@dataclass(frozen=True)
class NestedGeometry:
    """Packed ragged batch of square samples.

    Pair tensors are ``(cells, P, H, D)`` contiguous, masks ``(cells, P)``, and the
    bias is head-major ``(P, H, bias_values)`` with each sample's block laid out as
    ``(groups, query, key)``.  ``transposed`` means that the packed cell order is
    column-major (the ending-node form).
    """

    lengths: Tuple[int, ...]
    prefixes: int
    transposed: bool
    bias_groups: Tuple[int, ...] = ()
    bias_row_strides: Tuple[int, ...] = ()  # key-axis stride of each sample's bias rows (>= N_i; padded for alignment)

    def _cell_starts(self) -> List[int]:
        starts, at = [], 0
        for n in self.lengths:
            starts.append(at)
            at += n * n
        return starts

    def pair_views(self, tensor: Tensor) -> List[Tensor]:
        _, prefixes, heads, dim = tensor.shape
        cell = prefixes * heads * dim
        views = []
        for n, start in zip(self.lengths, self._cell_starts()):
            major, minor = n * cell, cell
            row_stride, col_stride = (minor, major) if self.transposed else (major, minor)
            views.append(
                tensor.as_strided(
                    (prefixes, n, n, heads, dim),
                    (heads * dim, row_stride, col_stride, dim, 1),
                    tensor.storage_offset() + start * cell,
                )
            )
        return views

    def mask_views(self, mask: Tensor) -> List[Tensor]:
        prefixes = mask.shape[1]
        views = []
        for n, start in zip(self.lengths, self._cell_starts()):
            major, minor = n * prefixes, prefixes
            row_stride, col_stride = (minor, major) if self.transposed else (major, minor)
            views.append(
                mask.as_strided((prefixes, n, n), (1, row_stride, col_stride), mask.storage_offset() + start * prefixes)
            )
        return views

    def bias_views(self, bias: Tensor) -> List[Tensor]:
        prefixes, heads, total = bias.shape
        row_strides = self.bias_row_strides or self.lengths
        views, at = [], 0
        for n, groups, row in zip(self.lengths, self.bias_groups, row_strides):
            views.append(
                bias.as_strided(
                    (prefixes, groups, heads, n, n), (heads * total, n * row, total, row, 1), bias.storage_offset() + at
                )
            )
            at += groups * n * row
        return views

    def lse_sizes(self, query: Tensor) -> List[Tuple[int, int, int, int]]:
        heads = query.shape[2]
        return [(self.prefixes, n, heads, n) for n in self.lengths]

    def canonical_pair(self, tensor: Tensor) -> Tensor:
        return tensor.contiguous()

    def canonical_bias(self, bias: Tensor) -> Tensor:
        return bias.contiguous()


_CHECK_DEVICE_STATUS = False


@contextmanager
def checked_device_status(enabled: bool = True):
    """Inside the block every forward and reverse call ends by synchronising with the device and reading the
    library's device-side status word; a kernel that gave up one of its bounded waits (its outputs are then
    undefined) raises ``RuntimeError`` and the word is cleared.  Off by default because of the synchronisation:
    production callers poll ``oops_b200.runtime.cabi.device_status()`` at a point where they synchronise anyway."""
    global _CHECK_DEVICE_STATUS
    previous, _CHECK_DEVICE_STATUS = _CHECK_DEVICE_STATUS, enabled
    try:
        yield
    finally:
        _CHECK_DEVICE_STATUS = previous


def _raise_if_device_failed(what: str) -> None:
    if not _CHECK_DEVICE_STATUS:
        return
    status = cabi.device_status(reset=True)
    if status:
        raise RuntimeError(
            f"triangle_attention {what}: a kernel recorded device status {status} "
            f"({cabi.library().oops_ta_status_string(status).decode()}); its results are undefined"
        )


def _current_stream_handle(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _workspace(nbytes: int, device: torch.device) -> Optional[Tensor]:
    return torch.empty(max(int(nbytes), 1), dtype=torch.uint8, device=device) if nbytes else None


def _raise_status(status: int, what: str) -> None:
    message = f"triangle_attention {what} failed: {cabi.status_message(status)}"
    if status in (cabi.STATUS_INVALID_ARGUMENT,):
        raise ValueError(message)
    if status in (cabi.STATUS_CUDA_ERROR, cabi.STATUS_DEVICE_TIMEOUT, cabi.STATUS_WORKSPACE_TOO_SMALL):
        raise RuntimeError(message)
    from ..._errors import OOpsUnsupportedError

    raise OOpsUnsupportedError(message)


def _split_lse(lse: Tensor, sizes: Sequence[Tuple[int, int, int, int]]) -> List[Tensor]:
    pieces, at = [], 0
    for size in sizes:
        count = size[0] * size[1] * size[2] * size[3]
        pieces.append(lse[at : at + count])
        at += count
    return pieces


def run_forward(
    geometry, query: Tensor, key: Tensor, value: Tensor, mask: Optional[Tensor], bias: Optional[Tensor], scale: float,
    flags: int, want_lse: bool,
) -> Tuple[Tensor, Optional[Tensor]]:
    """Launch the forward pass of every view; returns ``(out, lse)``."""
    lib = cabi.library()
    device = query.device
    out = torch.empty_like(query)
    if out.shape[-1] != 1 and out.stride(-1) != 1:
        out = torch.empty(query.shape, dtype=query.dtype, device=device)
    sizes = geometry.lse_sizes(query)
    lse = None
    if want_lse:
        lse = torch.empty(sum(b * r * h * c for b, r, h, c in sizes), dtype=torch.float32, device=device)
    lse_views = _split_lse(lse, sizes) if lse is not None else [None] * len(sizes)
    q_views, k_views, v_views = geometry.pair_views(query), geometry.pair_views(key), geometry.pair_views(value)
    o_views = geometry.pair_views(out)
    m_views = geometry.mask_views(mask) if mask is not None else [None] * len(q_views)
    b_views = geometry.bias_views(bias) if bias is not None else [None] * len(q_views)
    with torch.cuda.device(device):
        stream = _current_stream_handle(device)
        for q, k, v, o, m, b, l in zip(q_views, k_views, v_views, o_views, m_views, b_views, lse_views):
            problem = cabi.make_problem(q, k, v, m, b, scale, flags)
            status = lib.oops_ta_supported(cabi.byref(problem))
            if status:
                _raise_status(status, "forward")
            scratch = _workspace(lib.oops_ta_forward_workspace_bytes(cabi.byref(problem)), device)
            if scratch is not None:
                problem.workspace = scratch.data_ptr()
                problem.workspace_bytes = scratch.numel()
            out_pair = cabi.pair_of(o)
            status = lib.oops_ta_forward(
                cabi.byref(problem), cabi.byref(out_pair), None if l is None else l.data_ptr(), stream
            )
            if status:
                _raise_status(status, "forward")
        _raise_if_device_failed("forward")
    return out, lse


def backward_scratch_bytes(query, key, value, mask, bias, scale, flags, need) -> int:
    """Scratch bytes the reverse pass of one dense ``(B, R, C, H, D)`` problem needs for this gradient request."""
    lib = cabi.library()
    problem = cabi.make_problem(query, key, value, mask, bias, scale, flags)
    grads = cabi.Grads()
    marker = cabi.Pair(1, 0, 0, 0, 0)  # the size query looks at which pointers are set, not at what they point to
    none = cabi.Pair(None, 0, 0, 0, 0)
    grads.dq, grads.dk, grads.dv = (marker if need[0] else none, marker if need[1] else none, marker if need[2] else none)
    if need[3] and bias is not None:
        grads.dbias = 1
    return int(lib.oops_ta_backward_workspace_bytes(cabi.byref(problem), cabi.byref(grads)))


def run_backward(
    geometry, grad_out: Tensor, query: Tensor, key: Tensor, value: Tensor, mask: Optional[Tensor],
    bias: Optional[Tensor], out: Tensor, lse: Tensor, scale: float, flags: int, need: Sequence[bool],
    *, scratch: Optional[Tensor] = None, dbias_dtype: Optional[torch.dtype] = None,
) -> Tuple[Optional[Tensor], Optional[Tensor], Optional[Tensor], Optional[Tensor]]:
    """Launch the reverse pass of every view; returns ``(dq, dk, dv, dbias)``.

    ``scratch`` lends a caller-owned byte buffer to the call (it must be large enough for every view; without it one
    buffer per view is allocated).  ``dbias_dtype`` overrides the type of the bias gradient buffer: ``torch.float32``
    together with ``cabi.FLAG_DBIAS_F32`` in ``flags`` returns the unrounded f32 sums of a row-shared bias."""
    lib = cabi.library()
    device = query.device
    need_q, need_k, need_v, need_b = need
    need_b = need_b and bias is not None

    def like(t: Tensor) -> Tensor:
        g = torch.empty_like(t)
        if g.shape[-1] != 1 and g.stride(-1) != 1:
            g = torch.empty(t.shape, dtype=t.dtype, device=device)
        return g

    dq = like(query) if need_q else None
    dk = like(key) if need_k else None
    dv = like(value) if need_v else None
    dbias = torch.empty(bias.shape, dtype=dbias_dtype or bias.dtype, device=device) if need_b else None

    sizes = geometry.lse_sizes(query)
    lse_views = _split_lse(lse, sizes)
    count = len(sizes)
    views = lambda t: geometry.pair_views(t) if t is not None else [None] * count  # noqa: E731
    q_views, k_views, v_views = views(query), views(key), views(value)
    o_views, do_views = views(out), views(grad_out)
    dq_views, dk_views, dv_views = views(dq), views(dk), views(dv)
    m_views = geometry.mask_views(mask) if mask is not None else [None] * count
    b_views = geometry.bias_views(bias) if bias is not None else [None] * count
    db_views = geometry.bias_views(dbias) if dbias is not None else [None] * count
    with torch.cuda.device(device):
        stream = _current_stream_handle(device)
        for i in range(count):
            problem = cabi.make_problem(q_views[i], k_views[i], v_views[i], m_views[i], b_views[i], scale, flags)
            grads = cabi.Grads()
            grads.dq, grads.dk, grads.dv = (cabi.pair_of(dq_views[i]), cabi.pair_of(dk_views[i]),
                                            cabi.pair_of(dv_views[i]))
            if db_views[i] is not None:
                grads.dbias = db_views[i].data_ptr()
                (grads.dbias_sb, grads.dbias_sg, grads.dbias_sh, grads.dbias_sq, grads.dbias_sk) = db_views[i].stride()
            nbytes = lib.oops_ta_backward_workspace_bytes(cabi.byref(problem), cabi.byref(grads))
            buffer = scratch if scratch is not None and scratch.numel() >= nbytes else _workspace(nbytes, device)
            if buffer is not None:
                problem.workspace = buffer.data_ptr()
                problem.workspace_bytes = buffer.numel()
            out_pair, dout_pair = cabi.pair_of(o_views[i]), cabi.pair_of(do_views[i])
            status = lib.oops_ta_backward(
                cabi.byref(problem), cabi.byref(out_pair), cabi.byref(dout_pair), lse_views[i].data_ptr(),
                cabi.byref(grads), stream,
            )
            if status:
                _raise_status(status, "backward")
        _raise_if_device_failed("backward")
    return dq, dk, dv, dbias


class TriangleAttentionFunction(torch.autograd.Function):
    """``out = f(query, key, value, mask, bias)`` with a hand-written reverse pass."""

    @staticmethod
    def forward(ctx, query, key, value, mask, bias, scale, geometry, flags):
        needs_grad = any(ctx.needs_input_grad[i] for i in (0, 1, 2, 4))
        out, lse = run_forward(geometry, query, key, value, mask, bias, scale, flags, want_lse=needs_grad)
        ctx.set_materialize_grads(False)
        if needs_grad:
            ctx.save_for_backward(query, key, value, mask, bias, out, lse)
            ctx.scale, ctx.geometry, ctx.flags = scale, geometry, flags
        return out

    @staticmethod
    def backward(ctx, grad_out):
        if grad_out is None:
            return (None,) * 8
        query, key, value, mask, bias, out, lse = ctx.saved_tensors
        geometry = ctx.geometry
        # Saved-tensor hooks may hand back copies with other strides; the views are rebuilt from what arrives.
        query, key, value, out = (geometry.canonical_pair(t) for t in (query, key, value, out))
        grad_out = geometry.canonical_pair(grad_out.resolve_neg().to(query.dtype))
        if bias is not None:
            bias = geometry.canonical_bias(bias)
        if mask is not None and not isinstance(geometry, DenseGeometry):
            mask = mask.contiguous()
        lse = lse.contiguous()
        need = (ctx.needs_input_grad[0], ctx.needs_input_grad[1], ctx.needs_input_grad[2], ctx.needs_input_grad[4])
        dq, dk, dv, dbias = run_backward(
            geometry, grad_out, query, key, value, mask, bias, out, lse, ctx.scale, ctx.flags, need
        )
        return dq, dk, dv, None, dbias, None, None, None


# ----------------------------------------------------------------------------------------------
# Dispatcher route: torch.library custom ops with fake (meta) implementations, used under torch.compile and
# FakeTensorMode, where tensors carry no data pointers.  Takes the place of the reference's
# `ooperators::_triangle_attention_forward/_backward` ops and their `register_fake` shape functions
# (oops/attention/triangle/triton/ops.py:156-366).  Eager calls keep the direct autograd.Function above.
# ----------------------------------------------------------------------------------------------


def encode_geometry(geometry) -> List[int]:
    """Flatten a geometry into integers (custom-op schemas carry no Python objects)."""
    if isinstance(geometry, DenseGeometry):
        return []
    count = len(geometry.lengths)
    groups = geometry.bias_groups or (0,) * count
    rows = geometry.bias_row_strides or geometry.lengths
    return [geometry.prefixes, int(geometry.transposed), count, int(bool(geometry.bias_groups)), *geometry.lengths, *groups,
            *rows]


def decode_geometry(code: Sequence[int]):
    if len(code) == 0:
        return DenseGeometry()
    prefixes, transposed, count, has_bias = (int(v) for v in code[:4])
    lengths = tuple(int(v) for v in code[4 : 4 + count])
    groups = tuple(int(v) for v in code[4 + count : 4 + 2 * count]) if has_bias else ()
    rows = tuple(int(v) for v in code[4 + 2 * count : 4 + 3 * count]) if has_bias else ()
    return NestedGeometry(lengths=lengths, prefixes=prefixes, transposed=bool(transposed), bias_groups=groups,
                          bias_row_strides=rows)


@torch.library.custom_op("oops_b200::triangle_attention_forward", mutates_args=())
def _forward_op(
    query: Tensor, key: Tensor, value: Tensor, mask: Optional[Tensor], bias: Optional[Tensor], scale: float,
    geometry: List[int], flags: int, want_lse: bool,
) -> Tuple[Tensor, Tensor]:
    out, lse = run_forward(decode_geometry(geometry), query, key, value, mask, bias, scale, flags, want_lse)
    if lse is None:
        lse = torch.empty(0, dtype=torch.float32, device=query.device)
    return out, lse


@_forward_op.register_fake
def _forward_fake(query, key, value, mask, bias, scale, geometry, flags, want_lse):
    out = torch.empty_like(query)
    count = query.numel() // query.shape[-1] if want_lse else 0
    return out, query.new_empty((count,), dtype=torch.float32)


@torch.library.custom_op("oops_b200::triangle_attention_backward", mutates_args=())
def _backward_op(
    grad_out: Tensor, query: Tensor, key: Tensor, value: Tensor, mask: Optional[Tensor], bias: Optional[Tensor],
    out: Tensor, lse: Tensor, scale: float, geometry: List[int], flags: int, need: List[bool],
) -> Tuple[Tensor, Tensor, Tensor, Tensor]:
    geom = decode_geometry(geometry)
    query_given, key_given, value_given, bias_given = query, key, value, bias
    query, key, value, out = (geom.canonical_pair(t) for t in (query, key, value, out))
    grad_out = geom.canonical_pair(grad_out.resolve_neg().to(query.dtype))
    if bias is not None:
        bias = geom.canonical_bias(bias)
    if mask is not None and not isinstance(geom, DenseGeometry):
        mask = mask.contiguous()
    given = (query_given, key_given, value_given, bias_given)
    grads = run_backward(geom, grad_out, query, key, value, mask, bias, out, lse.contiguous(), scale, flags, need)
    empty = torch.empty(0, dtype=query.dtype, device=query.device)

    def laid_out_like(grad, operand):
        # the fake implementation promises the operand's own strides; a gradient computed on a re-laid copy
        # (unaligned or non-unit-stride operands) is copied into that layout
        if grad is None:
            return empty
        if operand is None or grad.stride() == operand.stride():
            return grad
        return torch.empty_like(operand).copy_(grad)

    return tuple(laid_out_like(g, operand) for g, operand in zip(grads, given))


@_backward_op.register_fake
def _backward_fake(grad_out, query, key, value, mask, bias, out, lse, scale, geometry, flags, need):
    def like(t, wanted):
        return torch.empty_like(t) if wanted and t is not None else query.new_empty((0,))

    return like(query, need[0]), like(key, need[1]), like(value, need[2]), like(bias, need[3])


def _dispatch_setup(ctx, inputs, output):
    query, key, value, mask, bias, scale, geometry, flags, _want = inputs
    out, lse = output
    ctx.save_for_backward(query, key, value, mask, bias, out, lse)
    ctx.scale, ctx.geometry, ctx.flags = scale, geometry, flags
    ctx.set_materialize_grads(False)


def _dispatch_backward(ctx, grad_out, _grad_lse):
    if grad_out is None:
        return (None,) * 9
    query, key, value, mask, bias, out, lse = ctx.saved_tensors
    need = [ctx.needs_input_grad[0], ctx.needs_input_grad[1], ctx.needs_input_grad[2],
            ctx.needs_input_grad[4] and bias is not None]
    dq, dk, dv, db = _backward_op(grad_out, query, key, value, mask, bias, out, lse, ctx.scale, ctx.geometry, ctx.flags, need)
    return (dq if need[0] else None, dk if need[1] else None, dv if need[2] else None, None, db if need[3] else None,
            None, None, None, None)


_forward_op.register_autograd(_dispatch_backward, setup_context=_dispatch_setup)


def _needs_dispatcher(*tensors: Optional[Tensor]) -> bool:
    if torch.compiler.is_compiling():
        return True
    from torch._subclasses.fake_tensor import is_fake

    return any(t is not None and is_fake(t) for t in tensors)


def apply(query, key, value, mask, bias, scale, geometry, flags=0) -> Tensor:
    if _needs_dispatcher(query, key, value, mask, bias):
        want_lse = torch.is_grad_enabled() and any(t is not None and t.requires_grad for t in (query, key, value, bias))
        out, _ = _forward_op(query, key, value, mask, bias, scale, encode_geometry(geometry), flags, want_lse)
        return out
    return TriangleAttentionFunction.apply(query, key, value, mask, bias, scale, geometry, flags)
