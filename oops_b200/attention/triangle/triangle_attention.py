"""``triangle_attention`` -- the operator entry point.

Same signature, argument meaning and error behaviour as
``oops/attention/triangle/triangle_attention.py:38-101`` in the reference; the
work below it is done by hand-written sm_100a kernels behind a C ABI
(``include/oops_ta.h``) instead of Triton.
"""

from __future__ import annotations

from contextlib import contextmanager
from math import prod
from typing import Optional, Tuple

import torch
from torch import Tensor

from ...runtime import cabi, require_no_forward_mode, require_same_device, unsupported
from ...runtime.nested_tensor import is_nested
from . import function as _function
from .function import DenseGeometry, NestedGeometry, checked_device_status

_OPERATOR = "triangle_attention"
_DTYPES = (torch.float16, torch.bfloat16, torch.float32)


def triangle_attention(
    query,
    key,
    value,
    mask=None,
    triangle_bias=None,
    *,
    scale: Optional[float] = None,
):
    r"""Row-wise triangle attention over the column axis of pair features.

    Each row is an independent softmax domain:
    ``out[.., r, q, h, :] = softmax_k(scale * <query[.., r, q, h], key[.., r, k, h]> + bias[.., r|0, h, q, k]) @ value``.

    Args:
        query: dense ``(*prefix, R, C, H, D)`` with ``1 <= D <= 256`` and non-empty
            dimensions, or a packed ragged batch (DanLing ``NestedTensor`` or the
            stand-in in ``oops_b200.runtime.nested_tensor``) of square
            ``(*prefix, N_i, N_i, H, D)`` elements.  Passing views whose two pair
            axes are swapped in memory gives the ending-node form without a copy.
        key, value: same shape, dtype, device and ragged topology as ``query``.
        mask: optional bool keep-mask broadcastable to ``(*prefix, R, C)``;
            ``False`` drops key column ``c`` of row ``r``.
        triangle_bias: optional additive bias ``(*prefix, R|1, H, C, C)`` in the
            q/k/v dtype or float32.
        scale: multiplies ``q.k`` before the bias is added; default ``D ** -0.5``.

    Returns:
        Attention values with the query's shape, dtype, device and memory layout
        (a ragged result keeps the query's topology).  Rows without a kept key
        return zero.

    Raises:
        ValueError: shapes, devices, dense/ragged representations or ragged
            topologies disagree.
        OOpsUnsupportedError: unsupported device, dtype, layout, empty size,
            launch limit, or forward-mode differentiation.
    """
    operands = {"query": query, "key": key, "value": value, "mask": mask, "triangle_bias": triangle_bias}
    packed = {name for name, operand in operands.items() if operand is not None and is_nested(operand)}
    pair_names = {"query", "key", "value"}
    if packed & pair_names and not pair_names <= packed:
        raise ValueError(_MIXED_QKV)
    if not packed & pair_names:
        if packed:
            raise ValueError("triangle_attention dense query/key/value cannot use NestedTensor mask or triangle_bias")
        require_no_forward_mode(_OPERATOR, query, key, value, triangle_bias)
        return _dense(query, key, value, mask, triangle_bias, scale)
    # a packed ragged batch: every optional operand that is given must be packed too
    for name, message in _DENSE_OPTIONAL_WITH_PACKED.items():
        if operands[name] is not None and name not in packed:
            raise ValueError(message)
    return _nested(query, key, value, mask, triangle_bias, scale)


_MIXED_QKV = "triangle_attention query, key, and value must all use the same NestedTensor layout"
_DENSE_OPTIONAL_WITH_PACKED = {
    "mask": "triangle_attention mask must use the same NestedTensor layout as nested query/key/value",
    "triangle_bias": "triangle_attention triangle_bias must use a compatible NestedTensor layout with nested "
    "query/key/value",
}


# ----------------------------------------------------------------------------------------------
# dense
# ----------------------------------------------------------------------------------------------


def _describe(tensor: Optional[Tensor]) -> Optional[str]:
    return None if tensor is None else f"{tuple(tensor.shape)} {tensor.dtype} {tensor.device}"


_FORCE_GENERIC = False
_SPLIT_REVERSE = False


@contextmanager
def layout_agnostic_kernels(enabled: bool = True):
    """Route calls inside the block to the layout-agnostic FFMA kernels even where the tcgen05
    kernels apply (used to test both kernel families on the same inputs)."""
    global _FORCE_GENERIC
    previous, _FORCE_GENERIC = _FORCE_GENERIC, enabled
    try:
        yield
    finally:
        _FORCE_GENERIC = previous


@contextmanager
def separate_reverse_kernels(enabled: bool = True):
    """Route the reverse pass of calls inside the block to the separate dQ and dK/dV kernels even where the
    single-pass kernel applies (used to test both on the same inputs)."""
    global _SPLIT_REVERSE
    previous, _SPLIT_REVERSE = _SPLIT_REVERSE, enabled
    try:
        yield
    finally:
        _SPLIT_REVERSE = previous


def _flags() -> int:
    # The f32 kernels use full-precision products in every mode, which satisfies both the
    # "ieee" and the relaxed "tf32" setting of torch.backends.cuda.matmul.fp32_precision.
    return (cabi.FLAG_FORCE_GENERIC if _FORCE_GENERIC else 0) | (cabi.FLAG_SPLIT_REVERSE if _SPLIT_REVERSE else 0)


def _require_bool_mask(mask: Optional[Tensor]) -> None:
    if mask is not None and mask.dtype is not torch.bool:
        raise unsupported(_OPERATOR, "requires a bool keep-mask", mask_dtype=mask.dtype)


def _right_aligned_broadcast(shape: Tuple[int, ...], target: Tuple[int, ...]) -> bool:
    """Whether ``shape`` expands to ``target`` under the usual trailing-axis alignment."""
    if len(shape) > len(target):
        return False
    padded = (1,) * (len(target) - len(shape)) + tuple(shape)
    return all(own in (1, want) for own, want in zip(padded, target))


def _check_dense_shapes(query, key, value, mask, triangle_bias) -> None:
    rank = query.dim()
    if rank < 4:
        raise ValueError(
            "triangle_attention query must be (*prefix, rows, cols, num_heads, head_size) of rank at least 4, "
            f"got rank {rank}"
        )
    if not (tuple(key.shape) == tuple(value.shape) == tuple(query.shape)):
        raise ValueError("triangle_attention query, key, and value must have the same shape")
    prefix, (rows, cols, num_heads) = tuple(query.shape[:-4]), tuple(query.shape[-4:-1])
    pair_shape = (*prefix, rows, cols)
    if mask is not None and not _right_aligned_broadcast(tuple(mask.shape), pair_shape):
        raise ValueError(
            f"triangle_attention mask shape {tuple(mask.shape)} must broadcast to the query's "
            f"(*prefix, rows, cols) = {pair_shape}"
        )
    if triangle_bias is not None:
        got = tuple(triangle_bias.shape)
        accepted = {(*prefix, groups, num_heads, cols, cols) for groups in (1, rows)}
        if got not in accepted:
            wanted = (*prefix, "rows|1", num_heads, cols, cols)
            raise ValueError(f"triangle_attention triangle_bias shape {got} must be {wanted}")


def _check_admission(query, key, value, mask, bias, what: str) -> None:
    """Device/dtype/size admission (the reference's supports_triangle_attention, generic.py:64-111)."""
    ok = (
        query.is_cuda
        and query.dtype in _DTYPES
        and key.dtype == query.dtype
        and value.dtype == query.dtype
        and 0 < query.shape[-1] <= 256
        and all(size > 0 for size in query.shape)
        and (bias is None or bias.dtype in (query.dtype, torch.float32))
    )
    if not ok:
        raise unsupported(
            _OPERATOR,
            what,
            query=_describe(query),
            key=_describe(key),
            value=_describe(value),
            mask=_describe(mask),
            triangle_bias=_describe(bias),
        )


def _unit_inner(tensor: Tensor) -> Tensor:
    tensor = tensor.resolve_neg().resolve_conj()
    return tensor if tensor.shape[-1] == 1 or tensor.stride(-1) == 1 else tensor.contiguous()


def _dense(query, key, value, mask, triangle_bias, scale):
    _check_dense_shapes(query, key, value, mask, triangle_bias)
    require_same_device(_OPERATOR, query, key, value, mask, triangle_bias)
    _require_bool_mask(mask)
    _check_admission(
        query, key, value, mask, triangle_bias,
        "requires CUDA float16/bfloat16/float32 q/k/v of one dtype and shape with head_size <= 256, "
        "a bool mask broadcastable to (*prefix, rows, cols), and a (*prefix, rows|1, num_heads, cols, cols) "
        "bias in the q/k/v dtype or float32",
    )
    lead_rank = query.dim() - 4  # axes in front of (rows, cols, num_heads, head_size)

    def as_batch(tensor: Tensor, keep: int = 4) -> Tensor:
        """Fold the leading axes of ``(*lead, <keep axes>)`` into one batch axis (a view where strides allow)."""
        lead = tensor.dim() - keep
        if lead == 1:
            return tensor
        return tensor.unsqueeze(0) if lead == 0 else tensor.flatten(0, lead - 1)

    q5 = _unit_inner(as_batch(query))
    # operands that are the same object stay the same object: the kernels then read one buffer
    k5 = q5 if key is query else _unit_inner(as_batch(key))
    v5 = q5 if value is query else k5 if value is key else _unit_inner(as_batch(value))
    rows, cols, head_size = q5.shape[1], q5.shape[2], q5.shape[4]
    mask3 = None if mask is None else as_batch(mask.expand(query.shape[:-2]), keep=2)
    bias5 = None
    if triangle_bias is not None:
        bias5 = as_batch(triangle_bias).resolve_neg().resolve_conj().contiguous()
        if bias5.element_size() == 2 and cols % 8 != 0:
            # 16-byte aligned bias rows (the TMA kernels need them): pad the key axis, then view the first `cols` keys
            bias5 = torch.nn.functional.pad(bias5, (0, -cols % 8))[..., :cols]
    scale = head_size**-0.5 if scale is None else float(scale)
    out = _function.apply(q5, k5, v5, mask3, bias5, scale, DenseGeometry(), _flags())
    # undoing the batch fold never needs a copy: it removes a unit axis or splits the leading one
    return out if lead_rank == 1 else out.squeeze(0) if lead_rank == 0 else out.unflatten(0, tuple(query.shape[:lead_rank]))


# ----------------------------------------------------------------------------------------------
# ragged (NestedTensor)
# ----------------------------------------------------------------------------------------------


def _packing_of(nested, ragged_axes: Tuple[int, ...], static_axes: Tuple[int, ...]) -> Optional[bool]:
    """Classify how a ragged container packs its elements.

    ``ragged_axes`` are the element axes that vary per sample in their canonical order (the last two are the pair
    or query/key axes) and ``static_axes`` the remaining element axes in storage order.  Returns ``False`` when the
    container packs exactly ``(*ragged_axes, *static_axes)``, ``True`` when it packs the same with the last two ragged
    axes exchanged (the ending-node order), ``None`` for anything else.
    """
    found = (tuple(nested.ragged_dims), tuple(nested.packed_dim_order))
    for exchanged in (False, True):
        axes = ragged_axes[:-2] + (ragged_axes[-1], ragged_axes[-2]) if exchanged else ragged_axes
        if found == (axes, axes + static_axes):
            return exchanged
    return None


def _canonical_nested_qkv(operand: str, nested) -> Tuple[Tensor, bool]:
    rank = nested.dim()  # element rank plus the batch axis
    if rank < 5 or not nested.batch_first:
        raise ValueError(f"triangle_attention nested {operand} elements must have shape (*prefix, N_i, N_i, H, D)")
    p = rank - 5
    transposed = _packing_of(nested, (p, p + 1), (*range(p), p + 2, p + 3))
    if transposed is None:
        raise unsupported(
            _OPERATOR,
            f"requires explicit canonical or transposed (*prefix, N_i, N_i, H, D) nested {operand} packing",
            ragged_dims=tuple(nested.ragged_dims),
            packed_dim_order=tuple(nested.packed_dim_order),
        )
    values = nested.concat
    heads_and_channels = tuple(values.shape[-2:])
    if values.dim() != p + 3 or min(heads_and_channels) <= 0:
        raise ValueError(f"triangle_attention nested {operand} must retain positive num_heads and head_size axes")
    return values, transposed


def _broadcast_nested_prefix(values: Tensor, prefix_shape: Tuple[int, ...], tail_rank: int) -> Tensor:
    """Expand the static prefix axes of packed values ``(cells, *own_prefix, *tail)`` to ``prefix_shape``."""
    split = values.dim() - tail_rank
    cells, own, tail = values.shape[0], tuple(values.shape[1:split]), tuple(values.shape[split:])
    wanted = tuple(prefix_shape)
    if not _right_aligned_broadcast(own, wanted):
        raise ValueError("triangle_attention nested mask and bias static prefixes must broadcast to the query prefix")
    aligned = (1,) * (len(wanted) - len(own)) + own
    return values.reshape(cells, *aligned, *tail).expand(cells, *wanted, *tail)


def _boundaries(nested, level) -> list:
    """Sample boundaries as Python integers along ragged axis ``level`` (None: the packed axis).

    A container that keeps its shapes on the host hands them over directly (no tensor round trip, and a traced
    graph stays free of data-dependent reads); otherwise the offset tensors are read back.
    """
    host = getattr(nested, "host_offsets", None)
    if host is not None:
        return [int(v) for v in host(level)]
    if level is None:
        return nested.packed_offsets(dtype=torch.int64).tolist()
    return nested.ragged_level_offsets(level, dtype=torch.int64).tolist()


def _steps(boundaries) -> list:
    return [boundaries[i + 1] - boundaries[i] for i in range(len(boundaries) - 1)]


def _sample_lengths(operand: str, nested) -> Tuple[int, ...]:
    """Per-sample N from the ragged offsets, with the reference's checks (nested.py:34-47)."""
    rows, packed = _boundaries(nested, 0), _boundaries(nested, None)
    if len(rows) <= 1:
        raise unsupported(_OPERATOR, "does not serve an empty NestedTensor batch")
    if len(packed) != len(rows):
        raise ValueError(f"{_OPERATOR} {operand} packed offsets must contain one boundary per sample")
    sizes = _steps(rows)
    for size in sizes:
        if size <= 0:
            raise unsupported(_OPERATOR, "requires every nested pair element to have N > 0")
    if _steps(packed) != [size * size for size in sizes]:
        raise ValueError(f"{_OPERATOR} {operand} token dims must be square (N, N) per sample")
    return tuple(int(size) for size in sizes)


def _nested_mask(mask, prefix_shape, transposed: bool, lengths) -> Tensor:
    rank = mask.dim()
    if rank < 3 or not mask.batch_first:
        raise ValueError("triangle_attention nested mask elements must have shape (*prefix, N_i, N_i)")
    p = rank - 3
    mask_transposed = _packing_of(mask, (p, p + 1), tuple(range(p)))
    if mask_transposed is None:
        raise unsupported(
            _OPERATOR,
            "requires explicit canonical or transposed (*prefix, N_i, N_i) nested mask packing",
            ragged_dims=tuple(mask.ragged_dims),
            packed_dim_order=tuple(mask.packed_dim_order),
        )
    if mask_transposed is not transposed:
        raise ValueError("triangle_attention nested mask must share q/k/v packed pair-axis orientation")
    values = mask.concat
    if values.dim() != p + 1:
        raise ValueError("triangle_attention nested mask must have flattened square pair storage")
    _require_bool_mask(values)
    if _sample_lengths("mask", mask) != tuple(lengths):
        raise ValueError("triangle_attention mask layout must match the query layout per sample")
    return _broadcast_nested_prefix(values, prefix_shape, 0)


def _nested_bias(triangle_bias, num_heads: int, prefix_shape, lengths) -> Tuple[Tensor, Tuple[int, ...], Tuple[int, ...]]:
    """Validate a ragged bias and return it head-major and query-major: ``(P, H, values)`` where each
    sample's block is ordered ``(group, query, key)``, plus the per-sample group counts.

    The reference reaches the same layout with ``movedim(0, -1).contiguous()`` for canonical biases and
    a per-sample permutation for transposed ones (triangle_attention.py:317-325, nested.py:325-335);
    here both are plain differentiable PyTorch views and one copy.
    """
    rank = triangle_bias.dim()
    if rank < 5 or not triangle_bias.batch_first:
        raise ValueError(
            "triangle_attention nested triangle_bias elements must have shape (*prefix, rows|1, H, N_i, N_i)"
        )
    p = rank - 5
    # element axes: p = group (rows|1), p + 1 = head, p + 2 = query, p + 3 = key.  A row-shared bias varies per sample
    # in its query/key axes only; a per-row bias also in its group axis.
    shared, transposed = True, _packing_of(triangle_bias, (p + 2, p + 3), (*range(p), p, p + 1))
    if transposed is None:
        shared, transposed = False, _packing_of(triangle_bias, (p, p + 2, p + 3), (*range(p), p + 1))
    if transposed is None:
        raise unsupported(
            _OPERATOR,
            "requires literal dense-order nested triangle_bias elements with canonical or transposed shared/full "
            "pair-axis ragged dimensions",
            ragged_dims=tuple(triangle_bias.ragged_dims),
            packed_dim_order=tuple(triangle_bias.packed_dim_order),
        )
    packed = triangle_bias.concat
    if shared and packed.shape[-2] != 1:
        raise ValueError("triangle_attention row-shared nested triangle_bias must have a unit group axis")
    if packed.shape[-1] != num_heads:
        raise unsupported(
            _OPERATOR, "requires packed triangle_bias num_heads matching q/k/v", triangle_bias=_describe(packed),
            num_heads=num_heads,
        )
    packed_offsets = _boundaries(triangle_bias, None)
    if len(packed_offsets) != len(lengths) + 1:
        raise ValueError("triangle_attention triangle_bias must have one packed boundary per sample")
    counts = _steps(packed_offsets)
    if shared:
        groups = tuple(1 for _ in lengths)
        if counts != [n * n for n in lengths]:
            raise ValueError("triangle_attention shared triangle_bias layout must match query per sample")
    else:
        group_offsets = _boundaries(triangle_bias, 0)
        if len(group_offsets) != len(lengths) + 1:
            raise ValueError("triangle_attention triangle_bias must have one packed boundary per sample")
        groups = tuple(int(g) for g in _steps(group_offsets))
        for g, n in zip(groups, lengths):
            if g != 1 and g != n:
                raise ValueError("triangle_attention triangle_bias group axis must be 1 or N_i per sample")
        if counts != [g * n * n for g, n in zip(groups, lengths)]:
            raise ValueError("triangle_attention triangle_bias query/key axes must both have length N_i per sample")
    values = packed.squeeze(-2) if shared else packed
    values = _broadcast_nested_prefix(values, tuple(prefix_shape), 1)  # (T, *prefix, H)
    values = values.reshape(values.shape[0], -1, num_heads).resolve_neg().resolve_conj()
    prefixes = values.shape[1]
    # 16-bit biases get 16-byte aligned rows (the TMA kernels need them): the key axis of each sample is padded
    row_strides = tuple((n + 7) // 8 * 8 if values.element_size() == 2 else n for n in lengths)
    if not transposed and row_strides == tuple(lengths):
        head_major = values.permute(1, 2, 0).contiguous()
    else:
        pieces, at = [], 0
        for n, g, row in zip(lengths, groups, row_strides):
            block = values[at : at + g * n * n].reshape(g, n, n, prefixes, num_heads)
            # stored order is (group, query, key) or, transposed, (group, key, query); target (P, H, group, query, key)
            block = block.permute(3, 4, 0, 2, 1) if transposed else block.permute(3, 4, 0, 1, 2)
            if row != n:
                block = torch.nn.functional.pad(block, (0, row - n))
            pieces.append(block.reshape(prefixes, num_heads, g * n * row))
            at += g * n * n
        head_major = torch.cat(pieces, dim=2).contiguous()
    return head_major, groups, row_strides


def _nested(query, key, value, mask, triangle_bias, scale):
    pair_operands = (("query", query), ("key", key), ("value", value))
    unpacked = [_canonical_nested_qkv(name, operand) for name, operand in pair_operands]
    (query_values, transposed), (key_values, _), (value_values, _) = unpacked
    require_no_forward_mode(
        _OPERATOR, query_values, key_values, value_values, None if triangle_bias is None else triangle_bias.concat
    )
    if any(values.shape[1:] != query_values.shape[1:] for values, _ in unpacked[1:]):
        raise ValueError(
            "triangle_attention nested query, key, and value must share static prefix, num_heads, and head_size"
        )
    if any(orientation is not transposed for _, orientation in unpacked[1:]):
        raise ValueError("triangle_attention nested query, key, and value must share packed pair-axis orientation")
    lengths = _sample_lengths("query", query)
    for operand, nested in (("key", key), ("value", value)):
        if _sample_lengths(operand, nested) != lengths or nested.concat.shape[0] != query_values.shape[0]:
            raise ValueError(f"triangle_attention {operand} layout must match the query layout per sample")
    if query_values.shape[0] <= 0:
        raise unsupported(_OPERATOR, "requires non-empty packed pair values")

    prefix_shape = tuple(query_values.shape[1:-2])
    prefixes = prod(prefix_shape)
    num_heads, head_size = query_values.shape[-2:]
    total_cells = query_values.shape[0]

    mask_values = None
    if mask is not None:
        mask_values = _nested_mask(mask, prefix_shape, transposed, lengths).reshape(total_cells, prefixes).contiguous()
    bias_values, groups, row_strides = None, (), ()
    if triangle_bias is not None:
        bias_values, groups, row_strides = _nested_bias(triangle_bias, num_heads, prefix_shape, lengths)
    require_same_device(_OPERATOR, query_values, key_values, value_values, mask_values, bias_values)
    _check_admission(
        query_values, key_values, value_values, mask_values, bias_values,
        "requires CUDA float16/bfloat16/float32 canonical/transposed packed NestedTensor q/k/v with "
        "head_size <= 256, a matching bool nested mask, and independently canonical/transposed "
        "nested triangle bias in the q/k/v dtype or float32",
    )

    def packed4(values: Tensor) -> Tensor:
        return values.resolve_neg().resolve_conj().reshape(total_cells, prefixes, num_heads, head_size).contiguous()

    q4 = packed4(query_values)
    k4 = q4 if key_values is query_values else packed4(key_values)
    v4 = q4 if value_values is query_values else k4 if value_values is key_values else packed4(value_values)
    geometry = NestedGeometry(
        lengths=lengths, prefixes=prefixes, transposed=transposed, bias_groups=tuple(groups),
        bias_row_strides=tuple(row_strides),
    )
    scale = head_size**-0.5 if scale is None else float(scale)
    out = _function.apply(q4, k4, v4, mask_values, bias_values, scale, geometry, _flags())
    return query.packed_like(out.reshape(total_cells, *prefix_shape, num_heads, head_size))


__all__ = ["triangle_attention", "layout_agnostic_kernels", "separate_reverse_kernels", "checked_device_status"]
