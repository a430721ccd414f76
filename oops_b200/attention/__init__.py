"""Attention operators (only the triangle-attention path is provided)."""

from .triangle import triangle_attention

__all__ = ["triangle_attention"]
