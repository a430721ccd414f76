"""Normalisation operators of the pair block (the reference's ``oops.normalization``)."""

from .layer_norm import layer_norm

__all__ = ["layer_norm"]
