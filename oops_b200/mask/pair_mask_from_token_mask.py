"""Pair validity from token validity, with the reference's call surface.

Mirrors ``oops/mask/pair_mask_from_token_mask.py:33-103`` of the reference: a dense mask ``(..., N)`` gives the bool
tensor ``mask[..., :, None] & mask[..., None, :]`` on any device (one broadcast AND, as in the reference); a packed
ragged batch of ``(N_i,)`` elements gives a packed batch of ``(N_i, N_i)`` elements and needs CUDA storage: its values
come from ``oops_ta_pair_mask_packed`` (``include/oops_ta.h``), one launch for the whole batch.  The result is what
``triangle_attention`` takes as ``mask``.  Outputs are not differentiable.
"""

from __future__ import annotations

import torch
from torch import Tensor

from ..runtime import cabi, unsupported
from ..runtime.nested_tensor import is_nested

_NAME = "pair_mask_from_token_mask"
_CELLS_PER_THREAD = 16  # launch extent unit of oops_ta_pair_mask_packed


def _square_elements(token_mask, values: Tensor, lengths):
    """A packed batch of (N_i, N_i) elements around `values`, of the container type of `token_mask`."""
    if hasattr(token_mask, "packed_with_square_lengths"):  # DanLing
        return token_mask.packed_with_square_lengths(values, torch.tensor(lengths, dtype=torch.int64))
    return type(token_mask)._from_parts(values, [(n, n) for n in lengths], (0, 1), (0, 1))


def _dense(token_mask: Tensor) -> Tensor:
    if token_mask.dim() == 0:
        raise ValueError(f"{_NAME} token_mask must have at least one dimension")
    valid = token_mask.bool()
    return valid.unsqueeze(-1) & valid.unsqueeze(-2)


def _packed_tokens(batch) -> Tensor:
    """The packed token bytes of a ragged batch of (N_i,) elements, after the checks the kernel relies on."""
    canonical = batch.batch_first and batch.dim() == 2 and tuple(batch.ragged_dims) == (0,) and tuple(batch.packed_dim_order) == (0,)
    if not canonical:
        raise ValueError(f"{_NAME} nested elements require canonical (N_i,) packing")
    if len(batch) == 0:
        raise unsupported(_NAME, "does not serve an empty NestedTensor wrapper batch without retained element rank")
    values = batch.concat
    refusals = (
        (values.is_complex(), "requires bool, integer, or floating-point packed values", {"dtype": values.dtype}),
        (values.dim() != 1 or not values.is_contiguous(), "requires contiguous one-dimensional packed token values",
         {"packed_shape": tuple(values.shape)}),
        (not values.is_cuda, "requires CUDA packed values", {"device": values.device}),
    )
    for refused, reason, context in refusals:
        if refused:
            raise unsupported(_NAME, reason, **context)
    return values.bool()


def pair_mask_from_token_mask(token_mask):
    """Outer conjunction of token validity; see the module docstring.  Nonzero values count as valid."""
    if not is_nested(token_mask):
        return _dense(token_mask)
    tokens = _packed_tokens(token_mask)

    if hasattr(token_mask, "host_offsets"):
        bounds = token_mask.host_offsets(0)
    else:
        bounds = token_mask.ragged_level_offsets(0, dtype=torch.int64).tolist()
    lengths = [hi - lo for lo, hi in zip(bounds[:-1], bounds[1:])]
    cells = sum(n * n for n in lengths)
    chunks = sum(n * ((n + _CELLS_PER_THREAD - 1) // _CELLS_PER_THREAD) for n in lengths)
    out = torch.empty(cells, dtype=torch.bool, device=tokens.device)
    if chunks:
        offsets = torch.tensor(bounds, dtype=torch.int64).to(tokens.device, non_blocking=True)
        lib = cabi.library()
        with torch.cuda.device(tokens.device):
            status = lib.oops_ta_pair_mask_packed(tokens.data_ptr(), offsets.data_ptr(), len(lengths), chunks, out.data_ptr(),
                                                  torch.cuda.current_stream(tokens.device).cuda_stream)
        if status:
            raise unsupported(_NAME, cabi.status_message(status), samples=len(lengths))
    return _square_elements(token_mask, out, lengths)
