"""Attention operators: triangle attention and the gated output step that follows it in a pair block."""

from .gate import gate_attention_output, triangle_attention_gated
from .triangle import triangle_attention

__all__ = ["triangle_attention", "gate_attention_output", "triangle_attention_gated"]
