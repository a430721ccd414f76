"""B200-native triangle attention with the call surface of OOps' ``oops`` package.

``import oops_b200 as oops`` gives ``oops.triangle_attention`` and
``oops.OOpsUnsupportedError`` with the reference's signature and error behaviour
(``oops/__init__.py:33,73`` in the reference re-exports the same two names).
"""

from ._errors import OOpsUnsupportedError
from .attention import triangle_attention
from .runtime.nested_tensor import NestedTensor

__all__ = ["OOpsUnsupportedError", "NestedTensor", "triangle_attention"]
