"""CPU oracle for the gated attention output.  TEST INFRASTRUCTURE ONLY.

Only the test-suite may import this module; nothing under ``oops_b200`` does.

It restates the reference's own PyTorch statement of the operator, ``_reference`` in
``tests/attention/gate/test_gate_attention_output.py:40-43`` (the same math as the composed fallback
``oops/attention/gate/composed.py:47-53``): the head-major attention values ``(*prefix, H, Q, D)`` are re-laid
token-major ``(*prefix, Q, H*D)``, multiplied by ``sigmoid(linear(single, gate_weight))`` and projected with
``output_weight``.  ``gated_values`` is the element-wise core alone, which is what the fused triangle-attention
epilogue produces.

Parity pin: ``tests/golden/gate.pt`` holds outputs and autograd gradients of the reference's ``_reference``
(lifted from its test file by ``tests/golden/make_golden_gate.py``); ``tests/test_oracle.py`` checks this module
against them.
"""

from __future__ import annotations

import torch
from torch import Tensor
from torch.nn import functional as F


def gated_values(attention: Tensor, gate_logits: Tensor, *, compute_dtype: torch.dtype = torch.float32) -> Tensor:
    """``sigmoid(gate_logits) * attention`` for two tensors of one shape (any layout), in ``compute_dtype``."""
    return torch.sigmoid(gate_logits.to(compute_dtype)) * attention.to(compute_dtype)


def gate_attention_output(attention: Tensor, single: Tensor, gate_weight: Tensor, output_weight: Tensor, *,
                          compute_dtype: torch.dtype = torch.float32) -> Tensor:
    """test_gate_attention_output.py:40-43; differentiable; returns ``compute_dtype`` of shape ``(*prefix, Q, O)``."""
    attention, single, gate_weight, output_weight = (t.to(compute_dtype) for t in (attention, single, gate_weight, output_weight))
    *prefix, heads, length, head_size = attention.shape
    token_major = attention.transpose(-3, -2).reshape(*prefix, length, heads * head_size)
    return F.linear(torch.sigmoid(F.linear(single, gate_weight)) * token_major, output_weight)
