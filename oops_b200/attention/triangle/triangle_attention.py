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
from .function import DenseGeometry, NestedGeometry

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
    if is_nested(query):
        if not is_nested(key) or not is_nested(value):
            raise ValueError("triangle_attention query, key, and value must all use the same NestedTensor layout")
        if mask is not None and not is_nested(mask):
            raise ValueError("triangle_attention mask must use the same NestedTensor layout as nested query/key/value")
        if triangle_bias is not None and not is_nested(triangle_bias):
            raise ValueError(
                "triangle_attention triangle_bias must use a compatible NestedTensor layout with nested query/key/value"
            )
        return _nested(query, key, value, mask, triangle_bias, scale)
    if is_nested(key) or is_nested(value):
        raise ValueError("triangle_attention query, key, and value must all use the same NestedTensor layout")
    if is_nested(mask) or is_nested(triangle_bias):
        raise ValueError("triangle_attention dense query/key/value cannot use NestedTensor mask or triangle_bias")
    require_no_forward_mode(_OPERATOR, query, key, value, triangle_bias)
    return _dense(query, key, value, mask, triangle_bias, scale)


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


def _check_dense_shapes(query, key, value, mask, triangle_bias) -> None:
    if query.dim() < 4:
        raise ValueError(
            "triangle_attention query must be (*prefix, rows, cols, num_heads, head_size) of rank at least 4, "
            f"got rank {query.dim()}"
        )
    if key.shape != query.shape or value.shape != query.shape:
        raise ValueError("triangle_attention query, key, and value must have the same shape")
    if mask is not None:
        target = tuple(query.shape[:-2])
        if mask.dim() > len(target) or any(
            size not in (1, extent) for size, extent in zip(reversed(mask.shape), reversed(target))
        ):
            raise ValueError(
                f"triangle_attention mask shape {tuple(mask.shape)} must broadcast to the query's "
                f"(*prefix, rows, cols) = {target}"
            )
    if triangle_bias is not None:
        *prefix, rows, cols, num_heads, _head_size = query.shape
        expected = (*prefix, "rows|1", num_heads, cols, cols)
        shape = tuple(triangle_bias.shape)
        if (
            triangle_bias.dim() != query.dim()
            or shape[: len(prefix)] != tuple(prefix)
            or shape[len(prefix)] not in (1, rows)
            or shape[len(prefix) + 1 :] != (num_heads, cols, cols)
        ):
            raise ValueError(f"triangle_attention triangle_bias shape {shape} must be {expected}")


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
    shape = query.shape
    batchless = query.dim() == 4
    prefixed = query.dim() > 5

    def batched(tensor: Tensor) -> Tensor:
        if batchless:
            return tensor.unsqueeze(0)
        return tensor.flatten(0, -5) if prefixed else tensor

    q5 = _unit_inner(batched(query))
    k5 = q5 if key is query else _unit_inner(batched(key))
    v5 = q5 if value is query else k5 if value is key else _unit_inner(batched(value))
    batch, rows, cols, _heads, head_size = q5.shape
    mask3 = None
    if mask is not None:
        mask3 = mask.expand(shape[:-2]).reshape(batch, rows, cols) if prefixed else mask.expand(shape[:-2])
        if batchless:
            mask3 = mask3.unsqueeze(0)
    bias5 = None
    if triangle_bias is not None:
        bias5 = batched(triangle_bias).resolve_neg().resolve_conj().contiguous()
        if bias5.element_size() == 2 and cols % 8 != 0:
            # 16-byte aligned bias rows (the TMA kernels need them): pad the key axis, then view the first `cols` keys
            bias5 = torch.nn.functional.pad(bias5, (0, -cols % 8))[..., :cols]
    scale = head_size**-0.5 if scale is None else float(scale)
    out = _function.apply(q5, k5, v5, mask3, bias5, scale, DenseGeometry(), _flags())
    if batchless:
        return out.squeeze(0)
    return out.reshape(shape) if prefixed else out


# ----------------------------------------------------------------------------------------------
# ragged (NestedTensor)
# ----------------------------------------------------------------------------------------------


def _canonical_nested_qkv(operand: str, nested) -> Tuple[Tensor, bool]:
    if not nested.batch_first or nested.dim() < 5:
        raise ValueError(f"triangle_attention nested {operand} elements must have shape (*prefix, N_i, N_i, H, D)")
    prefix_rank = nested.dim() - 5
    tail = (*range(prefix_rank), prefix_rank + 2, prefix_rank + 3)
    ragged, order = tuple(nested.ragged_dims), tuple(nested.packed_dim_order)
    canonical = ragged == (prefix_rank, prefix_rank + 1) and order == (prefix_rank, prefix_rank + 1, *tail)
    transposed = ragged == (prefix_rank + 1, prefix_rank) and order == (prefix_rank + 1, prefix_rank, *tail)
    if not canonical and not transposed:
        raise unsupported(
            _OPERATOR,
            f"requires explicit canonical or transposed (*prefix, N_i, N_i, H, D) nested {operand} packing",
            ragged_dims=ragged,
            packed_dim_order=order,
        )
    values = nested.concat
    if values.dim() != prefix_rank + 3 or values.shape[-2] <= 0 or values.shape[-1] <= 0:
        raise ValueError(f"triangle_attention nested {operand} must retain positive num_heads and head_size axes")
    return values, transposed


def _broadcast_nested_prefix(values: Tensor, prefix_shape: Tuple[int, ...], tail_rank: int) -> Tensor:
    own_prefix = tuple(values.shape[1 : values.dim() - tail_rank] if tail_rank else values.shape[1:])
    message = "triangle_attention nested mask and bias static prefixes must broadcast to the query prefix"
    try:
        broadcast_prefix = torch.broadcast_shapes(own_prefix, prefix_shape)
    except RuntimeError as error:
        raise ValueError(message) from error
    if tuple(broadcast_prefix) != tuple(prefix_shape):
        raise ValueError(message)
    tail = tuple(values.shape[-tail_rank:]) if tail_rank else ()
    return values.reshape(values.shape[0], *((1,) * (len(prefix_shape) - len(own_prefix))), *own_prefix, *tail).expand(
        values.shape[0], *prefix_shape, *tail
    )


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
    if not mask.batch_first or mask.dim() < 3:
        raise ValueError("triangle_attention nested mask elements must have shape (*prefix, N_i, N_i)")
    prefix_rank = mask.dim() - 3
    tail = tuple(range(prefix_rank))
    ragged, order = tuple(mask.ragged_dims), tuple(mask.packed_dim_order)
    canonical = ragged == (prefix_rank, prefix_rank + 1) and order == (prefix_rank, prefix_rank + 1, *tail)
    mask_transposed = ragged == (prefix_rank + 1, prefix_rank) and order == (prefix_rank + 1, prefix_rank, *tail)
    if not canonical and not mask_transposed:
        raise unsupported(
            _OPERATOR,
            "requires explicit canonical or transposed (*prefix, N_i, N_i) nested mask packing",
            ragged_dims=ragged,
            packed_dim_order=order,
        )
    if mask_transposed != transposed:
        raise ValueError("triangle_attention nested mask must share q/k/v packed pair-axis orientation")
    values = mask.concat
    if values.dim() != prefix_rank + 1:
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
    if not triangle_bias.batch_first or triangle_bias.dim() < 5:
        raise ValueError(
            "triangle_attention nested triangle_bias elements must have shape (*prefix, rows|1, H, N_i, N_i)"
        )
    prefix_rank = triangle_bias.dim() - 5
    ragged, order = tuple(triangle_bias.ragged_dims), tuple(triangle_bias.packed_dim_order)
    static_prefix = tuple(range(prefix_rank))
    shared_tail = (*static_prefix, prefix_rank, prefix_rank + 1)
    full_tail = (*static_prefix, prefix_rank + 1)
    if ragged == (prefix_rank + 2, prefix_rank + 3) and order == (*ragged, *shared_tail):
        shared, transposed = True, False
    elif ragged == (prefix_rank + 3, prefix_rank + 2) and order == (*ragged, *shared_tail):
        shared, transposed = True, True
    elif ragged == (prefix_rank, prefix_rank + 2, prefix_rank + 3) and order == (*ragged, *full_tail):
        shared, transposed = False, False
    elif ragged == (prefix_rank, prefix_rank + 3, prefix_rank + 2) and order == (*ragged, *full_tail):
        shared, transposed = False, True
    else:
        raise unsupported(
            _OPERATOR,
            "requires literal dense-order nested triangle_bias elements with canonical or transposed shared/full "
            "pair-axis ragged dimensions",
            ragged_dims=ragged,
            packed_dim_order=order,
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
    query_values, transposed = _canonical_nested_qkv("query", query)
    key_values, key_transposed = _canonical_nested_qkv("key", key)
    value_values, value_transposed = _canonical_nested_qkv("value", value)
    require_no_forward_mode(
        _OPERATOR, query_values, key_values, value_values, None if triangle_bias is None else triangle_bias.concat
    )
    if key_values.shape[1:] != query_values.shape[1:] or value_values.shape[1:] != query_values.shape[1:]:
        raise ValueError(
            "triangle_attention nested query, key, and value must share static prefix, num_heads, and head_size"
        )
    if key_transposed != transposed or value_transposed != transposed:
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


__all__ = ["triangle_attention", "layout_agnostic_kernels"]
