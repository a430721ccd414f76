"""CPU oracle for triangle attention.  TEST INFRASTRUCTURE ONLY.

This module is the checker, never the product: only the test-suite, the smoke
check and the ``cpu_baseline`` / ``--impl reference`` legs of the benchmark may
import it.  Nothing under ``oops_b200`` imports it.

It restates, in plain PyTorch on host cores, the math that the reference pins
its GPU kernels against:

* ``_reference`` in ``tests/attention/triangle/test_triangle_attention.py:42-58``
  (dense case): default scale ``D ** -0.5`` (:44), head-major transposition
  (:45-47), ``scores = (q @ k^T) * scale`` (:48), additive bias (:49-50), key
  keep-mask broadcast as ``mask[..., :, None, None, :]`` (:51), ``-inf`` fill and
  the all-zero scores for rows with no valid key (:53-54), softmax (:55),
  zeroing of masked probabilities (:57), ``P @ v`` and the transposition back
  (:58).
* ``_independent_nested_attention`` / ``_flatten_nested_attention`` (:148-169)
  for ragged batches: one dense evaluation per sample, packed by flattening the
  two pair axes row-major (canonical) or column-major (transposed) and
  concatenating samples.

The reference materialises the full ``[*, R, H, C, C]`` score tensor.  Rows are
independent softmax domains, so this restatement evaluates blocks of rows and
accumulates the row-shared bias gradient across blocks; results are identical
up to floating-point summation order of that one accumulation.

Parity pin: ``tests/golden/*.pt`` hold outputs of the reference's own
``_reference`` function (extracted from the reference test file by
``tests/golden/make_golden.py``); ``tests/test_oracle.py`` checks this module
against them.
"""

from __future__ import annotations

from typing import Optional, Sequence, Tuple

import torch
from torch import Tensor


def reference_dense(
    query: Tensor,
    key: Tensor,
    value: Tensor,
    mask: Optional[Tensor] = None,
    bias: Optional[Tensor] = None,
    scale: Optional[float] = None,
    *,
    compute_dtype: torch.dtype = torch.float32,
) -> Tensor:
    """Unblocked restatement (test_triangle_attention.py:42-58); differentiable.

    query/key/value: ``(*prefix, R, C, H, D)``; mask: bool broadcastable to
    ``(*prefix, R, C)``; bias: ``(*prefix, R|1, H, C, C)``.  Returns the
    ``compute_dtype`` result with the query's shape.
    """
    scale = query.shape[-1] ** -0.5 if scale is None else scale
    q = query.to(compute_dtype).transpose(-2, -3)
    k = key.to(compute_dtype).transpose(-2, -3)
    v = value.to(compute_dtype).transpose(-2, -3)
    scores = (q @ k.transpose(-1, -2)) * scale
    if bias is not None:
        scores = scores + bias.to(compute_dtype)
    keep = None if mask is None else mask.bool()[..., :, None, None, :]
    if keep is not None:
        scores = scores.masked_fill(~keep, float("-inf"))
        scores = torch.where(keep.any(dim=-1, keepdim=True), scores, torch.zeros_like(scores))
    probabilities = torch.softmax(scores, dim=-1)
    if keep is not None:
        probabilities = probabilities.masked_fill(~keep, 0.0)
    return (probabilities @ v).transpose(-2, -3)


def _row_block(rows: int, cols: int, heads: int, batch: int, itemsize: int, budget_bytes: int) -> int:
    per_row = max(1, batch * heads * cols * cols * itemsize)
    return max(1, min(rows, budget_bytes // per_row))


def forward(
    query: Tensor,
    key: Tensor,
    value: Tensor,
    mask: Optional[Tensor] = None,
    bias: Optional[Tensor] = None,
    scale: Optional[float] = None,
    *,
    compute_dtype: torch.dtype = torch.float32,
    budget_bytes: int = 1 << 30,
) -> Tensor:
    """Row-blocked forward for ``(B, R, C, H, D)`` inputs; returns ``compute_dtype``."""
    assert query.dim() == 5, "blocked oracle takes (B, R, C, H, D)"
    batch, rows, cols, heads, _ = query.shape
    block = _row_block(rows, cols, heads, batch, torch.empty((), dtype=compute_dtype).element_size(), budget_bytes)
    if mask is not None:
        mask = mask.expand(batch, rows, cols)
    pieces = []
    with torch.no_grad():
        for start in range(0, rows, block):
            stop = min(rows, start + block)
            b = None if bias is None else (bias if bias.shape[1] == 1 else bias[:, start:stop])
            m = None if mask is None else mask[:, start:stop]
            pieces.append(
                reference_dense(
                    query[:, start:stop], key[:, start:stop], value[:, start:stop], m, b, scale,
                    compute_dtype=compute_dtype,
                )
            )
    return torch.cat(pieces, dim=1)


def forward_backward(
    query: Tensor,
    key: Tensor,
    value: Tensor,
    mask: Optional[Tensor],
    bias: Optional[Tensor],
    grad_output: Tensor,
    scale: Optional[float] = None,
    *,
    compute_dtype: torch.dtype = torch.float32,
    budget_bytes: int = 1 << 30,
) -> Tuple[Tensor, Tensor, Tensor, Tensor, Optional[Tensor]]:
    """Row-blocked forward + reverse pass through autograd of the restatement.

    Returns ``(out, dq, dk, dv, dbias)`` in ``compute_dtype``.  ``dbias`` has the
    bias' own shape (row-shared biases receive the sum over rows).
    """
    assert query.dim() == 5, "blocked oracle takes (B, R, C, H, D)"
    batch, rows, cols, heads, _ = query.shape
    block = _row_block(rows, cols, heads, batch, torch.empty((), dtype=compute_dtype).element_size() * 4, budget_bytes)
    if mask is not None:
        mask = mask.expand(batch, rows, cols)
    shared = bias is not None and bias.shape[1] == 1
    out, dq, dk, dv, dbias_rows = [], [], [], [], []
    dbias_shared = None
    for start in range(0, rows, block):
        stop = min(rows, start + block)
        q = query[:, start:stop].detach().to(compute_dtype).requires_grad_(True)
        k = key[:, start:stop].detach().to(compute_dtype).requires_grad_(True)
        v = value[:, start:stop].detach().to(compute_dtype).requires_grad_(True)
        if bias is None:
            b = None
        else:
            b = (bias if shared else bias[:, start:stop]).detach().to(compute_dtype).requires_grad_(True)
        m = None if mask is None else mask[:, start:stop]
        with torch.enable_grad():
            o = reference_dense(q, k, v, m, b, scale, compute_dtype=compute_dtype)
            leaves = (q, k, v) if b is None else (q, k, v, b)
            grads = torch.autograd.grad(o, leaves, grad_output[:, start:stop].to(compute_dtype))
        out.append(o.detach())
        dq.append(grads[0])
        dk.append(grads[1])
        dv.append(grads[2])
        if b is not None:
            if shared:
                dbias_shared = grads[3] if dbias_shared is None else dbias_shared + grads[3]
            else:
                dbias_rows.append(grads[3])
    dbias = None
    if bias is not None:
        dbias = dbias_shared if shared else torch.cat(dbias_rows, dim=1)
    return torch.cat(out, 1), torch.cat(dq, 1), torch.cat(dk, 1), torch.cat(dv, 1), dbias


def nested_forward(
    queries: Sequence[Tensor],
    keys: Sequence[Tensor],
    values: Sequence[Tensor],
    masks: Optional[Sequence[Tensor]],
    biases: Optional[Sequence[Tensor]],
    scale: Optional[float] = None,
    *,
    compute_dtype: torch.dtype = torch.float32,
) -> Tuple[Tensor, ...]:
    """Per-sample dense evaluation (test_triangle_attention.py:148-157)."""
    count = len(queries)
    masks = (None,) * count if masks is None else masks
    biases = (None,) * count if biases is None else biases
    return tuple(
        reference_dense(q, k, v, m, b, scale, compute_dtype=compute_dtype)
        for q, k, v, m, b in zip(queries, keys, values, masks, biases)
    )


def flatten_nested(elements: Sequence[Tensor], *, transposed_pair_axes: bool = False) -> Tensor:
    """Packed order of a ragged batch (test_triangle_attention.py:160-169).

    Each element is ``(*prefix, N, N, H, D)``; its two pair axes are moved to the
    front (row-major, or column-major when ``transposed_pair_axes``), flattened
    into one cell axis, and the samples are concatenated along it.
    """
    values = []
    for element in elements:
        prefix_rank = element.dim() - 4
        first, second = prefix_rank, prefix_rank + 1
        if transposed_pair_axes:
            first, second = second, first
        order = (first, second, *range(prefix_rank), element.dim() - 2, element.dim() - 1)
        values.append(element.permute(order).flatten(0, 1))
    return torch.cat(values)


def flops(batch: int, rows: int, cols: int, heads: int, head_dim: int, *, backward: bool) -> float:
    """Algorithmic FLOPs: forward 4*B*R*H*C^2*D, reverse 10*B*R*H*C^2*D (five GEMMs)."""
    scores = float(batch) * rows * heads * cols * cols
    return scores * head_dim * (14.0 if backward else 4.0)
