"""B200-native triangle attention with the call surface of OOps' ``oops`` package.

``import oops_b200 as oops`` gives ``oops.triangle_attention``, ``oops.gate_attention_output``, ``oops.pair_mask_from_token_mask`` and
``oops.OOpsUnsupportedError`` with the reference's signatures and error behaviour
(``oops/__init__.py:33,73`` in the reference re-exports the same names), plus
``oops.triangle_attention_gated``, triangle attention with the gate of the following output
projection fused into its forward kernel.
"""

from ._errors import OOpsUnsupportedError
from .attention import gate_attention_output, pair_bias_attention, triangle_attention, triangle_attention_gated
from .mask import pair_mask_from_token_mask
from .normalization import layer_norm
from .pair import triangle_multiplication
from .runtime.nested_tensor import NestedTensor

__all__ = ["OOpsUnsupportedError", "NestedTensor", "triangle_attention", "gate_attention_output", "triangle_attention_gated",
           "pair_mask_from_token_mask", "layer_norm", "pair_bias_attention",
           "triangle_multiplication"]
