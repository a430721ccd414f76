"""Host-side helpers of the triangle-attention path.

Only the handful of helpers the operator entry point needs are restated here;
they mirror the behaviour of ``oops/runtime/dispatch.py`` in the reference
(error factory :514-526, same-device check :443, compile predicate :451,
forward-mode predicates :583-635).
"""

from __future__ import annotations

import torch
from torch import Tensor
from torch.autograd import forward_ad

from .._errors import OOpsUnsupportedError


def unsupported(operator: str, reason: str, **context: object) -> OOpsUnsupportedError:
    """Build the uniform ``"<operator> <reason> (k=v, ...)"`` unsupported error."""
    suffix = ""
    if context:
        suffix = " (" + ", ".join(f"{key}={value}" for key, value in context.items()) + ")"
    return OOpsUnsupportedError(f"{operator} {reason}{suffix}")


def is_compiling() -> bool:
    return torch.compiler.is_compiling()


def require_same_device(operator: str, *tensors: Tensor | None) -> None:
    devices = {tensor.device for tensor in tensors if tensor is not None}
    if len(devices) > 1:
        raise ValueError(f"{operator} operands must share one device, got {sorted(map(str, devices))}")


def require_shape(condition: bool, message: str) -> None:
    if not condition:
        raise ValueError(message)


def _functorch_jvp_active() -> bool:
    functorch = getattr(torch._C, "_functorch", None)
    if functorch is None:
        return False
    peek = getattr(functorch, "peek_interpreter_stack", None)
    if peek is None or peek() is None:
        return False
    get_stack = getattr(functorch, "get_interpreter_stack", None)
    stack = get_stack() if get_stack is not None else None
    jvp = getattr(getattr(functorch, "TransformType", None), "Jvp", None)
    if stack is None or jvp is None:
        return forward_ad._current_level >= 0
    return any(interpreter.key() == jvp for interpreter in stack) or forward_ad._current_level >= 0


def forward_mode_active(*tensors: Tensor | None) -> bool:
    """True when a dual tensor is among the operands or a ``torch.func.jvp`` transform is running."""
    if _functorch_jvp_active():
        return True
    if forward_ad._current_level < 0:
        return False
    return any(
        tensor is not None and isinstance(tensor, Tensor) and forward_ad.unpack_dual(tensor).tangent is not None
        for tensor in tensors
    )


def require_no_forward_mode(operator: str, *tensors: Tensor | None) -> None:
    if torch.compiler.is_compiling():  # the probe reads interpreter state a traced graph cannot hold
        return
    if forward_mode_active(*tensors):
        raise unsupported(
            operator,
            "does not support forward-mode AD",
            hint="use reverse-mode autograd or the equivalent Torch operation for a Jacobian-vector product",
        )


__all__ = [
    "unsupported", "is_compiling", "require_same_device", "require_shape", "forward_mode_active",
    "require_no_forward_mode",
]
