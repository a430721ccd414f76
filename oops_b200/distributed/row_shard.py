"""Row-sharded triangle attention across the GPUs of one node.

Every pair row is an independent softmax domain, so query, key, value, mask, the
output and their gradients are partitioned by row with no communication.  The
only coupled operand is the row-shared bias ``(B, 1, H, C, C)``: a row-sharded
model produces it sharded along its *query* axis (``bias[h, q, :]`` is a
projection of pair row ``q``), so it is all-gathered along that axis before the
local attention runs, and its gradient -- a partial sum over the local rows on
every rank -- is reduce-scattered back along the same axis.  The reference has no
multi-GPU code; this module is new.

Collectives go through ``torch.distributed`` (NCCL over NVLink/NVSwitch on GPUs,
gloo in the CPU tests).  The attention kernels only ever read the gathered bias
from the rank's own memory.

On GPUs the exchange is laid out so that nothing is copied around it and nothing is rounded twice:

* the shards are gathered head by head straight into the final ``(B, 1, H, C, C)`` buffer (within one head the ranks'
  query rows are consecutive blocks of memory);
* the reverse pass first runs the bias-gradient kernel alone, into an f32 buffer, and hands each head to a
  reduce-scatter that sums the ranks' f32 partial sums; the collectives run on the communication stream while the
  compute stream goes on with dQ, dK and dV (which reuse the row sums the first call left in the scratch buffer);
  the summed shard is rounded to the bias type once, at the end.
"""

from __future__ import annotations

from typing import Callable, Optional, Tuple

import torch
import torch.distributed as dist
from torch import Tensor

from ..attention.triangle import triangle_attention


def shard_bounds(rows: int, world_size: int, rank: int) -> Tuple[int, int]:
    """Half-open row range of ``rank``; rows must divide evenly so that the bias shards line up."""
    if rows % world_size != 0:
        raise ValueError(f"rows={rows} must be divisible by the number of ranks ({world_size})")
    per_rank = rows // world_size
    return rank * per_rank, (rank + 1) * per_rank


def _gather_into_place(shard: Tensor, group) -> Tensor:
    """All-gather a ``(B, 1, H, C/P, C)`` shard along the query axis into a new ``(B, 1, H, C, C)`` tensor, one
    collective per (batch, head): rank p's rows of a head are the p-th contiguous block of that head's plane."""
    world = dist.get_world_size(group)
    batch, groups, heads, own, cols = shard.shape
    shard = shard.contiguous()
    full = torch.empty((batch, groups, heads, world * own, cols), dtype=shard.dtype, device=shard.device)
    for b in range(batch):
        for g in range(groups):
            for h in range(heads):
                dist.all_gather_into_tensor(full[b, g, h].view(-1), shard[b, g, h].view(-1), group=group)
    return full


def _scatter_sum(full: Tensor, group, async_op: bool):
    """Reduce-scatter a ``(B, 1, H, C, C)`` tensor along the query axis, one collective per (batch, head); returns the
    ``(B, 1, H, C/P, C)`` sum shard and the pending work handles (empty unless ``async_op``)."""
    world = dist.get_world_size(group)
    batch, groups, heads, rows, cols = full.shape
    shard = torch.empty((batch, groups, heads, rows // world, cols), dtype=full.dtype, device=full.device)
    pending = []
    if dist.get_backend(group) == "gloo":  # gloo has no reduce_scatter_tensor
        summed = full.clone()
        dist.all_reduce(summed, group=group)
        rank = dist.get_rank(group)
        shard.copy_(summed[:, :, :, rank * (rows // world) : (rank + 1) * (rows // world)])
        return shard, pending
    for b in range(batch):
        for g in range(groups):
            for h in range(heads):
                work = dist.reduce_scatter_tensor(shard[b, g, h].view(-1), full[b, g, h].view(-1), group=group, async_op=async_op)
                if async_op:
                    pending.append(work)
    return shard, pending


class _GatherQueryAxis(torch.autograd.Function):
    """all-gather along the query axis (dim -2); reverse pass: reduce-scatter of the gradient.  Composable with any
    local operator (the CPU tests pair it with a PyTorch restatement); gradients are exchanged in the bias type."""

    @staticmethod
    def forward(ctx, shard: Tensor, group) -> Tensor:
        ctx.group = group
        return _gather_into_place(shard, group)

    @staticmethod
    def backward(ctx, grad_full: Tensor):
        shard, _ = _scatter_sum(grad_full.contiguous(), ctx.group, async_op=False)
        return shard, None


def gather_bias(bias_shard: Tensor, group=None) -> Tensor:
    """Differentiable all-gather of a ``(B, 1, H, C/P, C)`` bias shard into ``(B, 1, H, C, C)``."""
    return _GatherQueryAxis.apply(bias_shard, group)


class _RowShardedAttention(torch.autograd.Function):
    """Local attention over this rank's rows with the bias exchange folded in (CUDA, one dense problem)."""

    @staticmethod
    def forward(ctx, query, key, value, mask, bias_shard, scale, group, flags):
        from ..attention.triangle import function as fn

        bias = _gather_into_place(bias_shard, group)
        needs_grad = any(ctx.needs_input_grad[i] for i in (0, 1, 2, 4))
        out, lse = fn.run_forward(fn.DenseGeometry(), query, key, value, mask, bias, scale, flags, want_lse=needs_grad)
        ctx.set_materialize_grads(False)
        if needs_grad:
            ctx.save_for_backward(query, key, value, mask, bias, out, lse)
            ctx.scale, ctx.group, ctx.flags = scale, group, flags
        return out

    @staticmethod
    def backward(ctx, grad_out):
        from ..attention.triangle import function as fn
        from ..runtime import cabi

        if grad_out is None:
            return (None,) * 8
        query, key, value, mask, bias, out, lse = ctx.saved_tensors
        geometry = fn.DenseGeometry()
        query, key, value, out = (geometry.canonical_pair(t) for t in (query, key, value, out))
        grad_out = geometry.canonical_pair(grad_out.resolve_neg().to(query.dtype))
        need_q, need_k, need_v, need_b = (ctx.needs_input_grad[i] for i in (0, 1, 2, 4))
        device = query.device
        # One scratch buffer serves both calls, so that the second finds the row sums of the first.
        sizes = []
        if need_b:
            sizes.append(fn.backward_scratch_bytes(query, key, value, mask, bias, ctx.scale, ctx.flags | cabi.FLAG_DBIAS_F32,
                                                   (False, False, False, True)))
        if need_q or need_k or need_v:
            sizes.append(fn.backward_scratch_bytes(query, key, value, mask, bias, ctx.scale, ctx.flags,
                                                   (need_q, need_k, need_v, False)))
        scratch = torch.empty(max(sizes + [1]), dtype=torch.uint8, device=device)
        shard32, pending, reuse = None, [], 0
        if need_b:
            _, _, _, dbias32 = fn.run_backward(
                geometry, grad_out, query, key, value, mask, bias, out, lse, ctx.scale, ctx.flags | cabi.FLAG_DBIAS_F32,
                (False, False, False, True), scratch=scratch, dbias_dtype=torch.float32,
            )
            shard32, pending = _scatter_sum(dbias32, ctx.group, async_op=True)
            reuse = cabi.FLAG_REUSE_DELTA
        dq = dk = dv = None
        if need_q or need_k or need_v:
            dq, dk, dv, _ = fn.run_backward(
                geometry, grad_out, query, key, value, mask, bias, out, lse, ctx.scale, ctx.flags | reuse,
                (need_q, need_k, need_v, False), scratch=scratch,
            )
        for work in pending:
            work.wait()  # the compute stream waits for the collective; the host does not
        dbias_shard = None if shard32 is None else shard32.to(bias.dtype)
        return dq, dk, dv, None, dbias_shard, None, None, None


def row_sharded_triangle_attention(
    query: Tensor,
    key: Tensor,
    value: Tensor,
    mask: Optional[Tensor] = None,
    bias_shard: Optional[Tensor] = None,
    *,
    scale: Optional[float] = None,
    group=None,
    attention: Callable = triangle_attention,
) -> Tensor:
    """Starting-node triangle attention on this rank's rows.

    Args:
        query, key, value: this rank's rows, ``(B, R/P, C, H, D)``.
        mask: this rank's rows of the keep-mask, broadcastable to ``(B, R/P, C)``.
        bias_shard: this rank's query rows of the row-shared bias, ``(B, 1, H, C/P, C)``.
        group: process group (default: the world group).
        attention: the local operator (the CPU tests substitute a PyTorch restatement).

    Returns this rank's rows of the output.  In the reverse pass ``bias_shard.grad`` receives the
    bias gradient summed over the rows of *all* ranks for this rank's query rows.
    """
    fused_exchange = (
        attention is triangle_attention and bias_shard is not None and query.is_cuda and query.dim() == 5
        and query.dtype in (torch.float16, torch.bfloat16) and bias_shard.dtype == query.dtype and bias_shard.dim() == 5
        and bias_shard.shape[1] == 1 and not torch.compiler.is_compiling()
    )
    if not fused_exchange:
        bias = None if bias_shard is None else gather_bias(bias_shard, group)
        return attention(query, key, value, mask, bias, scale=scale)
    from ..attention.triangle.triangle_attention import (
        _check_admission, _check_dense_shapes, _flags, _require_bool_mask, _unit_inner,
    )

    world = dist.get_world_size(group)
    batch, rows, cols, heads, head_size = query.shape
    if tuple(bias_shard.shape) != (batch, 1, heads, cols // world, cols) or cols % world != 0:
        raise ValueError(
            f"row_sharded_triangle_attention bias_shard shape {tuple(bias_shard.shape)} must be "
            f"{(batch, 1, heads, 'cols/ranks', cols)} with cols divisible by the {world} ranks"
        )
    _check_dense_shapes(query, key, value, mask, None)
    _require_bool_mask(mask)
    _check_admission(query, key, value, mask, bias_shard, "requires CUDA float16/bfloat16 q/k/v of one dtype and shape")
    q5 = _unit_inner(query)
    k5 = q5 if key is query else _unit_inner(key)
    v5 = q5 if value is query else k5 if value is key else _unit_inner(value)
    mask3 = None if mask is None else mask.expand(batch, rows, cols)
    scale = head_size**-0.5 if scale is None else float(scale)
    return _RowShardedAttention.apply(q5, k5, v5, mask3, bias_shard, scale, group, _flags())


# ----------------------------------------------------------------------------------------------
# ending-node form under row sharding
# ----------------------------------------------------------------------------------------------


def _exchange_pair_axes(x: Tensor, group, rows_to_cols: bool) -> Tensor:
    """All-to-all between the two shardings of a pair tensor whose axes 1 and 2 are (row, column).

    ``rows_to_cols``: this rank's rows ``(B, R/P, C, *tail)`` become this rank's columns of all rows
    ``(B, R, C/P, *tail)``; otherwise the inverse.  Rank p owns the p-th contiguous block of the sharded axis."""
    world = dist.get_world_size(group)
    batch, a, b = x.shape[:3]
    tail = tuple(x.shape[3:])
    if rows_to_cols:
        if b % world != 0:
            raise ValueError(f"columns={b} must be divisible by the number of ranks ({world})")
        # piece for rank p: my rows, its block of columns
        send = x.reshape(batch, a, world, b // world, *tail).movedim(2, 0).contiguous()
        recv = torch.empty_like(send)
        dist.all_to_all_single(recv, send, group=group)
        # received piece p: rank p's rows, my block of columns
        return recv.movedim(0, 1).reshape(batch, world * a, b // world, *tail)
    if a % world != 0:
        raise ValueError(f"rows={a} must be divisible by the number of ranks ({world})")
    # piece for rank p: its block of rows, my columns
    send = x.reshape(batch, world, a // world, b, *tail).movedim(1, 0).contiguous()
    recv = torch.empty_like(send)
    dist.all_to_all_single(recv, send, group=group)
    # received piece p: my rows, rank p's block of columns
    return recv.movedim(0, 2).reshape(batch, a // world, world * b, *tail)


class _ExchangePairAxes(torch.autograd.Function):
    """Differentiable re-shard: the reverse pass is the inverse exchange of the gradient."""

    @staticmethod
    def forward(ctx, x: Tensor, group, rows_to_cols: bool) -> Tensor:
        ctx.group, ctx.rows_to_cols = group, rows_to_cols
        return _exchange_pair_axes(x, group, rows_to_cols)

    @staticmethod
    def backward(ctx, grad: Tensor):
        return _exchange_pair_axes(grad.contiguous(), ctx.group, not ctx.rows_to_cols), None, None


def reshard_rows_to_columns(x: Tensor, group=None) -> Tensor:
    """``(B, R/P, C, ...)`` (this rank's rows) -> ``(B, R, C/P, ...)`` (this rank's columns); differentiable."""
    return _ExchangePairAxes.apply(x, group, True)


def reshard_columns_to_rows(x: Tensor, group=None) -> Tensor:
    """``(B, R, C/P, ...)`` (this rank's columns) -> ``(B, R/P, C, ...)`` (this rank's rows); differentiable."""
    return _ExchangePairAxes.apply(x, group, False)


def row_sharded_ending_node_attention(
    query: Tensor,
    key: Tensor,
    value: Tensor,
    mask: Optional[Tensor] = None,
    bias_shard: Optional[Tensor] = None,
    *,
    scale: Optional[float] = None,
    group=None,
    attention: Callable = triangle_attention,
) -> Tensor:
    """Ending-node triangle attention for a pair tensor that is sharded by rows.

    The ending-node form attends along the *row* axis (the operator is called on the pair-axes transpose), so its
    softmax runs along the sharded axis: the pair tensors are first re-sharded to column ownership with one
    all-to-all each, the local call then runs on the transposed views (this rank's columns are its independent
    softmax domains; nothing is copied for the transpose, the kernels read the swapped strides), and the result is
    re-sharded back to rows.  No counterpart in the reference, which has no multi-GPU code.

    Args:
        query, key, value: this rank's rows ``(B, R/P, C, H, D)`` of the square pair tensors (R = C).
        mask: this rank's rows ``(B, R/P, C)`` of the keep-mask of the pair cells.
        bias_shard: this rank's query rows ``(B, 1, H, R/P, R)`` of the bias of the ending-node operator.

    Returns this rank's rows of the result, ``(B, R/P, C, H, D)``.
    """
    q, k, v = (reshard_rows_to_columns(t, group).transpose(1, 2) for t in (query, key, value))
    m = None
    if mask is not None:
        m = _exchange_pair_axes(mask.expand(query.shape[:3]).contiguous(), group, True).transpose(1, 2)
    out = row_sharded_triangle_attention(q, k, v, m, bias_shard, scale=scale, group=group, attention=attention)
    return reshard_columns_to_rows(out.transpose(1, 2), group)


__all__ = [
    "shard_bounds", "gather_bias", "row_sharded_triangle_attention", "reshard_rows_to_columns", "reshard_columns_to_rows",
    "row_sharded_ending_node_attention",
]
