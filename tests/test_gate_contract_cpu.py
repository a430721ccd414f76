"""Argument checking of gate_attention_output and triangle_attention_gated that needs no GPU
(reference: oops/attention/gate/_contract.py:27-48; tests/attention/gate/test_gate_attention_output.py:243-256)."""

from __future__ import annotations

import pytest
import torch

from oops_b200 import NestedTensor, OOpsUnsupportedError, gate_attention_output, triangle_attention_gated


def _operands():
    torch.manual_seed(0)
    return (torch.randn(2, 4, 9, 8), torch.randn(2, 9, 5), torch.randn(32, 5), torch.randn(7, 32))


def test_shape_contract_messages():
    attention, single, gate, weight = _operands()
    with pytest.raises(ValueError, match="attention must have layout"):
        gate_attention_output(attention[0, 0], single, gate, weight)
    with pytest.raises(ValueError, match="single must have layout"):
        gate_attention_output(attention, single[0], gate, weight)
    with pytest.raises(ValueError, match="rank-2 matrices"):
        gate_attention_output(attention, single, gate[0], weight)
    with pytest.raises(ValueError, match="share the attention leading axes"):
        gate_attention_output(attention, single[:, :8], gate, weight)
    with pytest.raises(ValueError, match=r"gate_weight must have shape"):
        gate_attention_output(attention, single, gate[:31], weight)
    with pytest.raises(ValueError, match="output_weight input channels"):
        gate_attention_output(attention, single, gate, weight[:, :31])


def test_cpu_and_ragged_operands_are_unsupported():
    attention, single, gate, weight = _operands()
    with pytest.raises(OOpsUnsupportedError, match="gate_attention_output requires CUDA"):
        gate_attention_output(attention, single, gate, weight)
    nested = NestedTensor([torch.randn(4, 3, 8)], ragged_dims=(1,))
    with pytest.raises(ValueError, match="nested attention requires a NestedTensor single"):
        gate_attention_output(nested, single, gate, weight)
    with pytest.raises(ValueError, match="dense attention cannot use a NestedTensor single"):
        gate_attention_output(attention, nested, gate, weight)


def test_gated_triangle_attention_checks():
    q = torch.randn(1, 3, 5, 2, 8)
    with pytest.raises(ValueError, match="gate must have the query's shape"):
        triangle_attention_gated(q, q, q, torch.randn(1, 3, 5, 2, 4))
    with pytest.raises(ValueError, match="rank"):
        triangle_attention_gated(q[0], q[0], q[0], q[0])
    with pytest.raises(OOpsUnsupportedError, match="requires CUDA"):
        triangle_attention_gated(q, q, q, q)
