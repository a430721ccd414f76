"""CPU restatement of token attention with pair bias for the parity tests.  TEST INFRASTRUCTURE: only tests/ may import
this module; the product path never does.

The reference's operator equals scaled-dot-product attention with the bias and the mask folded into an additive
attention mask (its composed form, ``oops/attention/pair_bias/composed.py:32-58``, calls
``F.scaled_dot_product_attention``).  The arithmetic is stated here explicitly, in float32 or float64;
``tests/test_pair_bias_cpu.py`` pins it against ``F.scaled_dot_product_attention`` itself.  Fully masked query rows
give zeros, as in the reference.
"""

from __future__ import annotations

from typing import Optional

import torch
from torch import Tensor


def pair_bias_attention(q: Tensor, k: Tensor, v: Tensor, key_mask: Optional[Tensor], bias: Optional[Tensor],
                        scale: Optional[float] = None, dtype=torch.float32) -> Tensor:
    """q, k, v: (..., H, N, D); key_mask: broadcastable to (..., 1, 1, N); bias: broadcastable to (..., H, N, N)."""
    q, k, v = q.to(dtype), k.to(dtype), v.to(dtype)
    s = q.shape[-1] ** -0.5 if scale is None else scale
    logits = torch.einsum("...qd,...kd->...qk", q, k) * s
    if bias is not None:
        logits = logits + bias.to(dtype)
    if key_mask is not None:
        logits = logits.masked_fill(~key_mask, float("-inf"))
    peak = logits.amax(dim=-1, keepdim=True)
    peak = torch.where(torch.isfinite(peak), peak, torch.zeros_like(peak))
    weights = torch.exp(logits - peak)
    total = weights.sum(dim=-1, keepdim=True)
    weights = torch.where(total > 0, weights / total.clamp_min(torch.finfo(dtype).tiny), torch.zeros_like(weights))
    return torch.einsum("...qk,...kd->...qd", weights, v)
