"""CPU restatement of layer normalisation for the parity tests.  TEST INFRASTRUCTURE: only tests/, the smoke entry and
the bench's CPU legs may import this module; the product path never does.

The reference checks its operator against ``F.layer_norm`` evaluated in float32 and cast to the activation dtype
(``tests/normalization/layer_norm/test_layer_norm.py:207-219``).  This module states that function's arithmetic
explicitly (mean, biased variance, ``rsqrt(var + eps)``, affine) so that the kernels are compared with formulas, and
``tests/test_layer_norm_oracle_cpu.py`` pins it against ``F.layer_norm`` itself, outputs and autograd gradients.
"""

from __future__ import annotations

from typing import Optional, Tuple

import torch
from torch import Tensor


def layer_norm(x: Tensor, weight: Optional[Tensor], bias: Optional[Tensor], eps: float = 1e-5, dtype=torch.float32) -> Tensor:
    """Normalised activations in `dtype` precision (float32 as in the reference's check, or float64)."""
    v = x.to(dtype)
    mean = v.mean(dim=-1, keepdim=True)
    centred = v - mean
    var = (centred * centred).mean(dim=-1, keepdim=True)
    out = centred * torch.rsqrt(var + eps)
    if weight is not None:
        out = out * weight.to(dtype)
    if bias is not None:
        out = out + bias.to(dtype)
    return out


def forward_backward(x: Tensor, weight: Optional[Tensor], bias: Optional[Tensor], upstream: Tensor, eps: float = 1e-5,
                     dtype=torch.float32) -> Tuple[Tensor, Tensor, Optional[Tensor], Optional[Tensor]]:
    """(y, dx, dweight, dbias) by the closed-form reverse pass; rows are the flattened leading axes."""
    width = x.shape[-1]
    v = x.to(dtype).reshape(-1, width)
    g = upstream.to(dtype).reshape(-1, width)
    mean = v.mean(dim=-1, keepdim=True)
    rstd = torch.rsqrt(((v - mean) ** 2).mean(dim=-1, keepdim=True) + eps)
    xhat = (v - mean) * rstd
    w = weight.to(dtype) if weight is not None else torch.ones(width, dtype=dtype)
    y = xhat * w + (bias.to(dtype) if bias is not None else 0)
    gw = g * w
    dx = rstd * (gw - gw.mean(dim=-1, keepdim=True) - xhat * (gw * xhat).mean(dim=-1, keepdim=True))
    dweight = (g * xhat).sum(dim=0) if weight is not None else None
    dbias = g.sum(dim=0) if bias is not None else None
    return y.reshape(x.shape), dx.reshape(x.shape), dweight, dbias
