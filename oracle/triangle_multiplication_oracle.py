"""CPU restatement of the triangle multiplicative update for the parity tests.  TEST INFRASTRUCTURE: only tests/ may
import this module; the product path never does.

Follows the reference's own check, ``_reference`` / ``_biased_reference`` in
``tests/pair/triangle_multiplication/test_triangle_multiplication.py:49-81`` (layer norm, masked gated projections,
contraction over the shared token, layer norm, gated output projection), with the contraction written as an explicit
einsum per direction and the layer norms taken from ``oracle/layer_norm_oracle.py``.
"""

from __future__ import annotations

import torch

from . import layer_norm_oracle


def _linear(x, weight, bias, dtype):
    out = x @ weight.to(dtype).T
    return out if bias is None else out + bias.to(dtype)


def triangle_multiplication(pair, mask, *, direction, input_norm_weight, input_norm_bias, left_value_weight, left_gate_weight,
                            right_value_weight, right_gate_weight, output_norm_weight, output_norm_bias, output_weight,
                            output_gate_weight, left_value_bias=None, left_gate_bias=None, right_value_bias=None,
                            right_gate_bias=None, output_bias=None, output_gate_bias=None, input_norm_eps=1e-5,
                            output_norm_eps=1e-5, dtype=torch.float32):
    x = layer_norm_oracle.layer_norm(pair, input_norm_weight, input_norm_bias, input_norm_eps, dtype)
    weight = 1.0 if mask is None else mask.to(dtype).unsqueeze(-1)
    left = weight * torch.sigmoid(_linear(x, left_gate_weight, left_gate_bias, dtype)) * _linear(x, left_value_weight, left_value_bias, dtype)
    right = weight * torch.sigmoid(_linear(x, right_gate_weight, right_gate_bias, dtype)) * _linear(x, right_value_weight, right_value_bias, dtype)
    if direction == "outgoing":
        update = torch.einsum("...ikh,...jkh->...ijh", left, right)
    else:
        update = torch.einsum("...kih,...kjh->...ijh", left, right)
    update = layer_norm_oracle.layer_norm(update, output_norm_weight, output_norm_bias, output_norm_eps, dtype)
    return _linear(update, output_weight, output_bias, dtype) * torch.sigmoid(_linear(x, output_gate_weight, output_gate_bias, dtype))
