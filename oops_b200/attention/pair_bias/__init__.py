"""Token attention with pair bias (the reference's ``oops.attention.pair_bias``), served by the triangle kernels."""

from .pair_bias_attention import pair_bias_attention

__all__ = ["pair_bias_attention"]
