"""Sigmoid-gated attention output: the step that follows triangle attention in a pair block."""

from .gate_attention_output import gate_attention_output, triangle_attention_gated

__all__ = ["gate_attention_output", "triangle_attention_gated"]
