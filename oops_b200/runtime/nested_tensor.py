"""Ragged-batch container used by the nested entry point.

The reference takes DanLing ``NestedTensor`` inputs (``danling.tensors``).  When
that package is importable it is used; otherwise this module provides a small
stand-in that implements only the surface the operator and its tests touch
(``oops/attention/triangle/triangle_attention.py:389-513`` and
``tests/attention/triangle/test_triangle_attention.py:66-169`` in the reference):

* ``NestedTensor(list_of_tensors, ragged_dims=...)`` -- elements of equal rank
  whose ``ragged_dims`` axes vary between samples;
* ``.concat`` -- the packed values: per sample the ragged axes come first (in
  ``packed_dim_order``), are flattened into one axis, and the samples are
  concatenated along it; the static axes follow;
* ``.packed_like(values)``, ``.ragged_dims``, ``.packed_dim_order``,
  ``.batch_first``, ``.dim()`` (element rank + 1);
* ``.ragged_level_offsets(0, dtype=)`` -- cumulative extents of the first ragged
  axis; ``.packed_offsets(dtype=)`` -- cumulative packed counts per sample;
* ``.transpose(a, b)`` -- metadata-only swap of two element axes;
* ``torch.unbind(nested)`` -- the per-sample tensors.

The operator itself is duck-typed (see ``is_nested``), so a real DanLing tensor
and this stand-in are interchangeable.
"""

from __future__ import annotations

from math import prod
from typing import Sequence, Tuple

import torch
from torch import Tensor

try:  # pragma: no cover - exercised only where danling is installed
    from danling.tensors import NestedTensor as _DanlingNestedTensor
except Exception:  # noqa: BLE001 - any import failure selects the stand-in
    _DanlingNestedTensor = None


class PackedNestedTensor:
    """Packed ragged batch; see the module docstring for the supported surface."""

    batch_first = True

    def __init__(self, tensors: Sequence[Tensor], ragged_dims: Sequence[int]):
        tensors = list(tensors)
        if not tensors:
            raise ValueError("NestedTensor needs at least one element")
        rank = tensors[0].dim()
        if any(t.dim() != rank for t in tensors):
            raise ValueError("NestedTensor elements must have one rank")
        ragged = tuple(int(d) % rank for d in ragged_dims)
        static = tuple(d for d in range(rank) if d not in ragged)
        self.ragged_dims: Tuple[int, ...] = ragged
        self.packed_dim_order: Tuple[int, ...] = (*ragged, *static)
        self._shapes = [tuple(t.shape) for t in tensors]
        pieces = [t.permute(self.packed_dim_order).flatten(0, len(ragged) - 1) for t in tensors]
        self._values = torch.cat(pieces, dim=0)

    # -- construction helpers -------------------------------------------------------------
    @classmethod
    def _from_parts(cls, values: Tensor, shapes, ragged_dims, packed_dim_order) -> "PackedNestedTensor":
        self = cls.__new__(cls)
        self._values = values
        self._shapes = [tuple(s) for s in shapes]
        self.ragged_dims = tuple(ragged_dims)
        self.packed_dim_order = tuple(packed_dim_order)
        return self

    def packed_like(self, values: Tensor) -> "PackedNestedTensor":
        if values.shape[0] != self._values.shape[0]:
            raise ValueError("packed values must keep the packed length")
        return self._from_parts(values, self._shapes, self.ragged_dims, self.packed_dim_order)

    # -- metadata -------------------------------------------------------------------------
    @property
    def concat(self) -> Tensor:
        return self._values

    def dim(self) -> int:
        return len(self._shapes[0]) + 1

    @property
    def device(self):
        return self._values.device

    @property
    def dtype(self):
        return self._values.dtype

    def __len__(self) -> int:
        return len(self._shapes)

    def host_offsets(self, level: int | None = None) -> list:
        """Sample boundaries as Python integers: along ragged axis ``level``, or of the packed axis when None.

        The shapes live on the host, so callers that only need lengths (the operator's admission checks, a traced
        graph) read them here without building a tensor and reading it back.
        """
        sizes = [0]
        for shape in self._shapes:
            if level is None:
                extent = 1
                for d in self.ragged_dims:
                    extent = extent * shape[d]
            else:
                extent = shape[self.ragged_dims[level]]
            sizes.append(sizes[-1] + extent)
        return sizes

    def ragged_level_offsets(self, level: int = 0, dtype=torch.int64) -> Tensor:
        return torch.tensor(self.host_offsets(level), dtype=dtype)

    def packed_offsets(self, dtype=torch.int64) -> Tensor:
        return torch.tensor(self.host_offsets(None), dtype=dtype)

    # -- views ----------------------------------------------------------------------------
    def transpose(self, first: int, second: int) -> "PackedNestedTensor":
        rank = self.dim()
        a, b = first % rank - 1, second % rank - 1
        if a < 0 or b < 0:
            raise ValueError("the batch axis of a NestedTensor cannot be transposed")

        def swap(d: int) -> int:
            return b if d == a else a if d == b else d

        shapes = []
        for shape in self._shapes:
            shape = list(shape)
            shape[a], shape[b] = shape[b], shape[a]
            shapes.append(tuple(shape))
        return self._from_parts(
            self._values, shapes, tuple(swap(d) for d in self.ragged_dims), tuple(swap(d) for d in self.packed_dim_order)
        )

    def unbind(self) -> Tuple[Tensor, ...]:
        order = self.packed_dim_order
        inverse = [order.index(d) for d in range(len(order))]
        parts, start = [], 0
        for shape in self._shapes:
            ragged_extent = prod(shape[d] for d in self.ragged_dims)
            block = self._values[start : start + ragged_extent]
            start += ragged_extent
            parts.append(block.reshape(*(shape[d] for d in order)).permute(inverse))
        return tuple(parts)

    @classmethod
    def __torch_function__(cls, func, types, args=(), kwargs=None):
        kwargs = kwargs or {}
        if func is torch.unbind:
            return args[0].unbind()
        return NotImplemented


NestedTensor = _DanlingNestedTensor if _DanlingNestedTensor is not None else PackedNestedTensor


def is_nested(value: object) -> bool:
    """Duck-typed test used by the operator: a packed ragged batch of either flavour."""
    if value is None or isinstance(value, Tensor):
        return False
    return all(hasattr(value, name) for name in ("concat", "ragged_dims", "packed_dim_order", "packed_like"))


__all__ = ["NestedTensor", "PackedNestedTensor", "is_nested"]
