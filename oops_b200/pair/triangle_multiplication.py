"""Triangle multiplicative update of pair features, composed from this library's layer norm and library GEMMs.

Mirrors the call surface of the reference's ``triangle_multiplication``
(``oops/pair/triangle_multiplication/triangle_multiplication.py:45-141``) for dense pairs ``(*prefix, N, N, C)``:

    x      = layer_norm(pair)                                        (this library's kernels)
    left   = mask * sigmoid(x Wlg^T + blg) * (x Wlv^T + blv)         right likewise
    update = sum_k left[i, k] * right[j, k]   ("outgoing")   or   sum_k left[k, i] * right[k, j]   ("incoming")
    out    = (layer_norm(update) Wo^T + bo) * sigmoid(x Wog^T + bog)

The two layer norms run on ``oops_ta_layer_norm_forward/_backward``; the six projections and the O(N^3) contraction
are plain GEMMs and go to the vendor library through ``torch`` (``F.linear``, ``torch.matmul``), as does the
element-wise gating; autograd composes the reverse pass.  No kernel of the contraction itself is built here.  Ragged
(NestedTensor) pairs raise ``OOpsUnsupportedError``.
"""

from __future__ import annotations

from typing import Optional

import torch
from torch import Tensor
from torch.nn import functional as F

from ..normalization import layer_norm
from ..runtime import require_no_forward_mode, require_same_device, unsupported
from ..runtime.nested_tensor import is_nested

_NAME = "triangle_multiplication"


def triangle_multiplication(pair, pair_mask: Optional[Tensor] = None, *, direction: str = "outgoing",
                            input_norm_weight: Tensor, input_norm_bias: Tensor, left_value_weight: Tensor,
                            left_gate_weight: Tensor, right_value_weight: Tensor, right_gate_weight: Tensor,
                            output_norm_weight: Tensor, output_norm_bias: Tensor, output_weight: Tensor,
                            output_gate_weight: Tensor, left_value_bias: Optional[Tensor] = None,
                            left_gate_bias: Optional[Tensor] = None, right_value_bias: Optional[Tensor] = None,
                            right_gate_bias: Optional[Tensor] = None, output_bias: Optional[Tensor] = None,
                            output_gate_bias: Optional[Tensor] = None, input_norm_eps: float = 1e-5,
                            output_norm_eps: float = 1e-5):
    """Incoming or outgoing triangle multiplicative update; see the module docstring."""
    if direction not in ("incoming", "outgoing"):
        raise ValueError(f"{_NAME} direction must be 'incoming' or 'outgoing', got {direction!r}")
    if is_nested(pair) or is_nested(pair_mask):
        raise unsupported(_NAME, "serves dense pairs only (NestedTensor pairs are not built)")
    tensors = (pair, pair_mask, input_norm_weight, input_norm_bias, left_value_weight, left_gate_weight, right_value_weight,
               right_gate_weight, output_norm_weight, output_norm_bias, output_weight, output_gate_weight, left_value_bias,
               left_gate_bias, right_value_bias, right_gate_bias, output_bias, output_gate_bias)
    require_no_forward_mode(_NAME, *tensors)
    require_same_device(_NAME, *tensors)
    if pair.dim() < 3 or pair.shape[-2] != pair.shape[-3]:
        raise ValueError(f"{_NAME} pair must have shape (*prefix, N, N, C) with a square token grid")
    channels = pair.shape[-1]
    hidden = left_value_weight.shape[0]
    expected = {"left_value_weight": (left_value_weight, (hidden, channels)), "left_gate_weight": (left_gate_weight, (hidden, channels)),
                "right_value_weight": (right_value_weight, (hidden, channels)), "right_gate_weight": (right_gate_weight, (hidden, channels)),
                "output_weight": (output_weight, (channels, hidden)), "output_gate_weight": (output_gate_weight, (channels, channels)),
                "input_norm_weight": (input_norm_weight, (channels,)), "input_norm_bias": (input_norm_bias, (channels,)),
                "output_norm_weight": (output_norm_weight, (hidden,)), "output_norm_bias": (output_norm_bias, (hidden,))}
    for name, (tensor, shape) in expected.items():
        if tuple(tensor.shape) != shape:
            raise ValueError(f"{_NAME} {name} must have shape {shape}, got {tuple(tensor.shape)}")
    if not pair.is_cuda:
        raise unsupported(_NAME, "requires CUDA pairs", device=pair.device)

    x = layer_norm(pair, channels, input_norm_weight, input_norm_bias, input_norm_eps)
    weight = 1.0 if pair_mask is None else pair_mask.to(x.dtype).unsqueeze(-1)
    left = weight * torch.sigmoid(F.linear(x, left_gate_weight.to(x.dtype), _cast(left_gate_bias, x))) * \
        F.linear(x, left_value_weight.to(x.dtype), _cast(left_value_bias, x))
    right = weight * torch.sigmoid(F.linear(x, right_gate_weight.to(x.dtype), _cast(right_gate_bias, x))) * \
        F.linear(x, right_value_weight.to(x.dtype), _cast(right_value_bias, x))
    # channel-major (..., H, N, N) operands of one batched GEMM per prefix element
    if direction == "outgoing":
        a, b = left.movedim(-1, -3), right.movedim(-1, -3).transpose(-1, -2)   # a[h, i, k], b[h, k, j] = right[j, k, h]
    else:
        a, b = left.movedim(-1, -3).transpose(-1, -2), right.movedim(-1, -3)   # a[h, i, k] = left[k, i, h], b[h, k, j]
    update = torch.matmul(a, b).movedim(-3, -1)
    update = layer_norm(update.contiguous(), hidden, output_norm_weight, output_norm_bias, output_norm_eps)
    out = F.linear(update, output_weight.to(x.dtype), _cast(output_bias, x))
    return out * torch.sigmoid(F.linear(x, output_gate_weight.to(x.dtype), _cast(output_gate_bias, x)))


def _cast(bias: Optional[Tensor], like: Tensor) -> Optional[Tensor]:
    return None if bias is None else bias.to(like.dtype)
