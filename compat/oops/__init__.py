"""``import oops`` for hosts that must keep the reference's import path.

Put this directory's parent (``compat/``) on ``PYTHONPATH`` and the names of the reference's ``oops`` package that this
library serves resolve to the B200 implementations (``oops/__init__.py:33,73`` in the reference re-exports the same
names).  Everything else the reference exports is absent: an attribute error, not a silent stand-in.  The directory is
not on the path by default, so an installed reference and this library can live in one environment.
"""

from oops_b200 import (  # noqa: F401
    NestedTensor,
    OOpsUnsupportedError,
    gate_attention_output,
    layer_norm,
    pair_bias_attention,
    pair_mask_from_token_mask,
    triangle_attention,
    triangle_multiplication,
)

__all__ = ["OOpsUnsupportedError", "NestedTensor", "triangle_attention", "gate_attention_output", "pair_mask_from_token_mask", "layer_norm", "pair_bias_attention", "triangle_multiplication"]
