"""Attention operators: triangle attention, the gated output step that follows it in a pair block, and token attention
with pair bias on the same kernels."""

from .gate import gate_attention_output, triangle_attention_gated
from .pair_bias import pair_bias_attention
from .triangle import triangle_attention

__all__ = ["triangle_attention", "gate_attention_output", "triangle_attention_gated", "pair_bias_attention"]
