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


class _GatherQueryAxis(torch.autograd.Function):
    """all-gather along the query axis (dim -2); reverse pass: reduce-scatter of the gradient."""

    @staticmethod
    def forward(ctx, shard: Tensor, group) -> Tensor:
        world = dist.get_world_size(group)
        ctx.group, ctx.world = group, world
        shard = shard.contiguous()
        flat = torch.empty(world * shard.numel(), dtype=shard.dtype, device=shard.device)
        dist.all_gather_into_tensor(flat, shard.view(-1), group=group)
        stacked = flat.view(world, *shard.shape)
        # (P, B, 1, H, C/P, C) -> (B, 1, H, P * C/P, C)
        return stacked.permute(1, 2, 3, 0, 4, 5).reshape(*shard.shape[:3], world * shard.shape[3], shard.shape[4])

    @staticmethod
    def backward(ctx, grad_full: Tensor):
        world, group = ctx.world, ctx.group
        b, g, h, c, k = grad_full.shape
        stacked = grad_full.reshape(b, g, h, world, c // world, k).permute(3, 0, 1, 2, 4, 5).contiguous()
        shard = torch.empty(stacked.shape[1:], dtype=grad_full.dtype, device=grad_full.device)
        if dist.get_backend(group) == "gloo":  # gloo has no reduce_scatter_tensor
            dist.all_reduce(stacked, group=group)
            shard.copy_(stacked[dist.get_rank(group)])
        else:
            dist.reduce_scatter_tensor(shard.view(-1), stacked.view(-1), group=group)
        return shard, None


def gather_bias(bias_shard: Tensor, group=None) -> Tensor:
    """Differentiable all-gather of a ``(B, 1, H, C/P, C)`` bias shard into ``(B, 1, H, C, C)``."""
    return _GatherQueryAxis.apply(bias_shard, group)


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
    bias = None if bias_shard is None else gather_bias(bias_shard, group)
    return attention(query, key, value, mask, bias, scale=scale)


__all__ = ["shard_bounds", "gather_bias", "row_sharded_triangle_attention"]
