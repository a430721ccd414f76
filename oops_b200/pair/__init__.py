"""Pair-representation updates (the reference's ``oops.pair``)."""

from .triangle_multiplication import triangle_multiplication

__all__ = ["triangle_multiplication"]
