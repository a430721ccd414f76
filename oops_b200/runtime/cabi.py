"""ctypes binding of liboops_ta_sm100.so (the C ABI declared in include/oops_ta.h).

The library is the only compute path: if it cannot be loaded the operator raises,
it never falls back to PyTorch math.
"""

from __future__ import annotations

import ctypes
from ctypes import POINTER, Structure, byref, c_char_p, c_float, c_int, c_int32, c_int64, c_uint32, c_uint64, c_void_p
from pathlib import Path
from typing import Optional

import torch
from torch import Tensor

ABI_VERSION = 1
F32, F16, BF16 = 0, 1, 2
FLAG_FORCE_GENERIC = 1
FLAG_SPLIT_REVERSE = 4
FLAG_DBIAS_F32 = 8
FLAG_REUSE_DELTA = 16

STATUS_OK = 0
STATUS_INVALID_ARGUMENT = 1
STATUS_WORKSPACE_TOO_SMALL = 6
STATUS_CUDA_ERROR = 7
STATUS_DEVICE_TIMEOUT = 8

DTYPE_CODE = {torch.float32: F32, torch.float16: F16, torch.bfloat16: BF16}

LIB_PATH = Path(__file__).resolve().parent.parent / "lib" / "liboops_ta_sm100.so"

EXPORTS = (
    "oops_ta_abi_version", "oops_ta_status_string", "oops_ta_last_error", "oops_ta_supported",
    "oops_ta_uses_tensor_path", "oops_ta_forward_workspace_bytes", "oops_ta_backward_workspace_bytes",
    "oops_ta_forward", "oops_ta_backward", "oops_ta_launch_count", "oops_ta_device_status",
    "oops_ta_forward_static", "oops_ta_forward_static_capacity", "oops_ta_selftest_wait_limit",
    "oops_ta_forward_gated", "oops_ta_gate_forward", "oops_ta_gate_backward", "oops_ta_pair_mask_packed", "oops_ta_layer_norm_backward_workspace_bytes", "oops_ta_layer_norm_forward",
    "oops_ta_layer_norm_backward",
)


class Pair(Structure):
    _fields_ = [("ptr", c_void_p), ("sb", c_int64), ("sr", c_int64), ("sc", c_int64), ("sh", c_int64)]


class Problem(Structure):
    _fields_ = [
        ("abi_version", c_uint32), ("flags", c_uint32), ("dtype", c_int32), ("bias_dtype", c_int32),
        ("batch", c_int32), ("rows", c_int32), ("cols", c_int32), ("heads", c_int32), ("head_dim", c_int32),
        ("bias_groups", c_int32), ("scale", c_float), ("reserved", c_int32),
        ("q", Pair), ("k", Pair), ("v", Pair),
        ("mask", c_void_p), ("mask_sb", c_int64), ("mask_sr", c_int64), ("mask_sc", c_int64),
        ("bias", c_void_p), ("bias_sb", c_int64), ("bias_sg", c_int64), ("bias_sh", c_int64),
        ("bias_sq", c_int64), ("bias_sk", c_int64),
        ("workspace", c_void_p), ("workspace_bytes", c_uint64),
    ]


class Grads(Structure):
    _fields_ = [
        ("dq", Pair), ("dk", Pair), ("dv", Pair),
        ("dbias", c_void_p), ("dbias_sb", c_int64), ("dbias_sg", c_int64), ("dbias_sh", c_int64),
        ("dbias_sq", c_int64), ("dbias_sk", c_int64),
    ]


_lib: Optional[ctypes.CDLL] = None


def library() -> ctypes.CDLL:
    """Load the shared library once; raise if it is missing or does not match the header."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m oops_b200.csrc.build` "
            "(triangle_attention has no other compute path)"
        )
    lib = ctypes.CDLL(str(LIB_PATH))
    for name in EXPORTS:
        if not hasattr(lib, name):
            raise RuntimeError(f"{LIB_PATH} does not export {name}")
    lib.oops_ta_abi_version.restype = c_int
    lib.oops_ta_status_string.restype = c_char_p
    lib.oops_ta_status_string.argtypes = [c_int]
    lib.oops_ta_last_error.restype = c_char_p
    lib.oops_ta_supported.restype = c_int
    lib.oops_ta_supported.argtypes = [POINTER(Problem)]
    lib.oops_ta_uses_tensor_path.restype = c_int
    lib.oops_ta_uses_tensor_path.argtypes = [POINTER(Problem), c_int]
    lib.oops_ta_forward_workspace_bytes.restype = c_uint64
    lib.oops_ta_forward_workspace_bytes.argtypes = [POINTER(Problem)]
    lib.oops_ta_backward_workspace_bytes.restype = c_uint64
    lib.oops_ta_backward_workspace_bytes.argtypes = [POINTER(Problem), POINTER(Grads)]
    lib.oops_ta_forward.restype = c_int
    lib.oops_ta_forward.argtypes = [POINTER(Problem), POINTER(Pair), c_void_p, c_void_p]
    lib.oops_ta_backward.restype = c_int
    lib.oops_ta_backward.argtypes = [POINTER(Problem), POINTER(Pair), POINTER(Pair), c_void_p, POINTER(Grads), c_void_p]
    lib.oops_ta_forward_static.restype = c_int
    lib.oops_ta_forward_static.argtypes = [POINTER(Problem), POINTER(Pair), c_void_p, c_void_p]
    lib.oops_ta_forward_static_capacity.restype = c_uint64
    lib.oops_ta_launch_count.restype = c_uint64
    lib.oops_ta_forward_gated.restype = c_int
    lib.oops_ta_forward_gated.argtypes = [POINTER(Problem), POINTER(Pair), POINTER(Pair), POINTER(Pair), c_void_p, c_void_p]
    lib.oops_ta_gate_forward.restype = c_int
    lib.oops_ta_gate_forward.argtypes = [c_int] * 6 + [POINTER(Pair)] * 3 + [c_void_p]
    lib.oops_ta_gate_backward.restype = c_int
    lib.oops_ta_gate_backward.argtypes = [c_int] * 6 + [POINTER(Pair)] * 5 + [c_void_p]
    lib.oops_ta_pair_mask_packed.restype = c_int
    lib.oops_ta_pair_mask_packed.argtypes = [c_void_p, c_void_p, c_int32, c_int64, c_void_p, c_void_p]
    lib.oops_ta_layer_norm_backward_workspace_bytes.restype = c_uint64
    lib.oops_ta_layer_norm_backward_workspace_bytes.argtypes = [c_int64, c_int32]
    lib.oops_ta_layer_norm_forward.restype = c_int
    lib.oops_ta_layer_norm_forward.argtypes = [c_int, c_int, c_int64, c_int32, c_void_p, c_int64, c_void_p, c_void_p, c_float,
                                               c_void_p, c_int64, c_void_p, c_void_p, c_void_p]
    lib.oops_ta_layer_norm_backward.restype = c_int
    lib.oops_ta_layer_norm_backward.argtypes = [c_int, c_int, c_int64, c_int32, c_void_p, c_int64, c_void_p, c_int64, c_void_p,
                                                c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_uint64,
                                                c_void_p]
    lib.oops_ta_selftest_wait_limit.restype = c_int
    lib.oops_ta_selftest_wait_limit.argtypes = [c_void_p]
    lib.oops_ta_device_status.restype = c_int
    lib.oops_ta_device_status.argtypes = [c_int]
    if lib.oops_ta_abi_version() != ABI_VERSION:
        raise RuntimeError(f"{LIB_PATH} has ABI {lib.oops_ta_abi_version()}, the binding expects {ABI_VERSION}")
    _lib = lib
    return lib


def status_message(status: int) -> str:
    lib = library()
    text = lib.oops_ta_status_string(status).decode()
    detail = lib.oops_ta_last_error().decode()
    return f"{text}: {detail}" if detail else text


def pair_of(tensor: Optional[Tensor]) -> Pair:
    """Describe a 5-D ``(B, R, C, H, D)`` tensor view whose last stride is 1."""
    if tensor is None:
        return Pair(None, 0, 0, 0, 0)
    assert tensor.dim() == 5 and (tensor.shape[-1] == 1 or tensor.stride(-1) == 1)
    sb, sr, sc, sh, _ = tensor.stride()
    return Pair(tensor.data_ptr(), sb, sr, sc, sh)


def make_problem(
    q: Tensor, k: Tensor, v: Tensor, mask: Optional[Tensor], bias: Optional[Tensor], scale: float, flags: int = 0
) -> Problem:
    """Fill a Problem from 5-D q/k/v views, a 3-D bool mask view and a 5-D bias view."""
    batch, rows, cols, heads, head_dim = q.shape
    problem = Problem()
    problem.abi_version = ABI_VERSION
    problem.flags = flags
    problem.dtype = DTYPE_CODE.get(q.dtype, -1)
    problem.batch, problem.rows, problem.cols, problem.heads, problem.head_dim = batch, rows, cols, heads, head_dim
    problem.scale = float(scale)
    problem.q, problem.k, problem.v = pair_of(q), pair_of(k), pair_of(v)
    if mask is not None:
        assert mask.dtype == torch.bool and mask.dim() == 3
        problem.mask = mask.data_ptr()
        problem.mask_sb, problem.mask_sr, problem.mask_sc = mask.stride()
    if bias is not None:
        assert bias.dim() == 5
        problem.bias_groups = bias.shape[1]
        problem.bias_dtype = DTYPE_CODE.get(bias.dtype, -1)
        problem.bias = bias.data_ptr()
        (problem.bias_sb, problem.bias_sg, problem.bias_sh, problem.bias_sq, problem.bias_sk) = bias.stride()
    else:
        problem.bias_groups = 0
        problem.bias_dtype = problem.dtype
    return problem


def device_status(reset: bool = True) -> int:
    """Synchronise and return the device-side status word (0 = ok, 8 = a bounded wait gave up)."""
    return int(library().oops_ta_device_status(1 if reset else 0))


def launch_count() -> int:
    return int(library().oops_ta_launch_count())


__all__ = [
    "ABI_VERSION", "EXPORTS", "LIB_PATH", "Pair", "Problem", "Grads", "library", "status_message", "pair_of",
    "make_problem", "launch_count", "device_status", "byref", "FLAG_FORCE_GENERIC", "FLAG_SPLIT_REVERSE", "FLAG_DBIAS_F32",
    "FLAG_REUSE_DELTA", "DTYPE_CODE",
]
