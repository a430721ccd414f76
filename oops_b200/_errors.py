"""Errors raised by the operators (mirrors oops/_errors.py:29-36 of the reference)."""

from __future__ import annotations


class OOpsUnsupportedError(NotImplementedError):
    """An operator cannot serve the requested device, dtype, layout, size domain,
    launch limit or differentiation mode.  Inconsistent arguments raise
    ``ValueError`` instead.  Unsupported calls always raise; there is no fallback."""
