"""Token attention with an additive pair bias, on the triangle-attention kernels.

The reference's ``pair_bias_attention`` (``oops/attention/pair_bias/pair_bias_attention.py:57-147``) is the sister
operator of triangle attention: head-major ``(*prefix, S, H, Q, D)`` queries, one softmax domain per prefix element,
group and head, an additive bias ``(*prefix, S|1, H|1, Q, K)`` and a bool keep-mask over keys.  With ``Q == K`` that is
triangle attention on a pair tensor whose rows are the groups: the head-major layout is a stride pattern of the same
``(B, R, C, H, D)`` problem, so the call below hands permuted *views* to ``triangle_attention`` and the tcgen05 kernels
read them in place (no copies of q, k, v or of the result).

Served: dense operands of rank 3 (``H, Q, D``), 4 (``S, H, Q, D``) or more (prefix axes), equal query and key
lengths, a key mask ``(*prefix, S|1, K)`` (optionally with unit query and head axes as in the reference), a bias
per group or shared by the groups, with its own heads or broadcast over them, reverse-mode gradients of q, k, v and
the bias.  The rest of the reference's contract raises ``OOpsUnsupportedError``: different query and key lengths,
masks with a query axis, singleton query / key bias axes, an f32 bias with 16-bit operands, NestedTensor operands and
the grouped / segmented variants.
"""

from __future__ import annotations

from typing import Optional

import torch
from torch import Tensor

from ...runtime import require_no_forward_mode, require_same_device, unsupported
from ...runtime.nested_tensor import is_nested
from ..triangle.triangle_attention import triangle_attention

_NAME = "pair_bias_attention"


def pair_bias_attention(query, key, value, mask: Optional[Tensor] = None, pair_bias: Optional[Tensor] = None, *,
                        scale: Optional[float] = None):
    """Scaled dot-product attention with an optional additive pair bias; see the module docstring."""
    if any(is_nested(t) for t in (query, key, value, mask, pair_bias)):
        raise unsupported(_NAME, "serves dense operands only (NestedTensor variants are not built)")
    require_no_forward_mode(_NAME, query, key, value, pair_bias)
    require_same_device(_NAME, query, key, value, mask, pair_bias)
    if query.dim() < 3:
        raise ValueError(f"{_NAME} query must have at least rank 3 (heads, tokens, channels)")
    if key.shape != value.shape or key.dim() != query.dim() or key.dtype != query.dtype or value.dtype != query.dtype:
        raise ValueError(f"{_NAME} key and value must match each other and the query's rank and dtype")
    rank = query.dim()
    # (*prefix, S, H, Q, D): rank 3 omits prefix and group, rank 4 the prefix
    lead = (1, 1) if rank == 3 else (1,) if rank == 4 else ()
    q5, k5, v5 = (t.reshape(*lead, *t.shape) if lead else t for t in (query, key, value))
    prefix = q5.shape[:-4]
    groups, heads, tokens, dim = q5.shape[-4:]
    if k5.shape[:-2] != q5.shape[:-2] or k5.shape[-1] != dim:
        raise ValueError(f"{_NAME} key and value must share the query's prefix, groups, heads and channels")
    if k5.shape[-2] != tokens:
        raise unsupported(_NAME, "serves equal query and key lengths only", query_length=tokens, key_length=k5.shape[-2])
    batch = 1
    for extent in prefix:
        batch *= extent

    def pairs(t: Tensor) -> Tensor:  # (*prefix, S, H, N, D) -> (B, S, N, H, D), a view whenever the prefix flattens
        return t.reshape(batch, groups, heads, tokens, dim).permute(0, 1, 3, 2, 4)

    key_mask = None
    if mask is not None:
        m = mask
        if m.dim() == rank:  # unit head axis before the query axis
            if m.shape[-3] != 1:
                raise unsupported(_NAME, "serves a mask head axis only of size 1", mask_shape=tuple(mask.shape))
            m = m.squeeze(-3)
        if m.dim() == rank - 1:
            if m.shape[-2] != 1:
                raise unsupported(_NAME, "serves key masks only (a mask with a query axis is not built)", mask_shape=tuple(mask.shape))
            m = m.squeeze(-2)
        if m.dim() != rank - 2 or m.shape[-1] != tokens:
            raise ValueError(f"{_NAME} mask must have shape (*batch_prefix, group|1, key_len) matching query/key")
        m = m.reshape(*lead, *m.shape) if lead else m
        if m.shape[:-2] != prefix or m.shape[-2] not in (1, groups):
            raise ValueError(f"{_NAME} mask must have shape (*batch_prefix, group|1, key_len) matching query/key")
        key_mask = m.bool().reshape(batch, m.shape[-2], tokens).expand(batch, groups, tokens)

    bias5 = None
    if pair_bias is not None:
        if pair_bias.dim() != rank:
            raise ValueError(f"{_NAME} pair_bias must have the query's rank: (*batch_prefix, group|1, num_heads|1, query, key)")
        b = pair_bias.reshape(*lead, *pair_bias.shape) if lead else pair_bias
        if (b.shape[:-4] != prefix or b.shape[-4] not in (1, groups) or b.shape[-3] not in (1, heads)
                or b.shape[-2] not in (1, tokens) or b.shape[-1] not in (1, tokens)):
            raise ValueError(f"{_NAME} pair_bias must have shape (*batch_prefix, group|1, num_heads|1, query_length|1, key_len|1)")
        if b.shape[-2] != tokens or b.shape[-1] != tokens:
            raise unsupported(_NAME, "does not serve singleton query or key bias axes", pair_bias_shape=tuple(pair_bias.shape))
        if b.dtype != query.dtype:
            raise unsupported(_NAME, "requires the bias in the dtype of query, key and value", bias_dtype=b.dtype)
        # broadcast heads are materialised by the operator's own layout step; autograd sums the gradient back
        bias5 = b.reshape(batch, b.shape[-4], b.shape[-3], tokens, tokens).expand(batch, b.shape[-4], heads, tokens, tokens)

    out = triangle_attention(pairs(q5), pairs(k5), pairs(v5), key_mask, bias5, scale=scale)
    return out.permute(0, 1, 3, 2, 4).reshape(query.shape)
