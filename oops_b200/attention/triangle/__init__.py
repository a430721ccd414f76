"""Triangle attention over the pair representation."""

from .triangle_attention import triangle_attention

__all__ = ["triangle_attention"]
