"""The C-ABI library loads without a GPU and exports every symbol the header declares."""

from __future__ import annotations

import ctypes
import re
from pathlib import Path

from oops_b200.runtime import cabi

ROOT = Path(__file__).resolve().parent.parent


def _declared_symbols():
    text = (ROOT / "include" / "oops_ta.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(oops_ta_[a-z_0-9]+)\s*\(", text)))


def test_header_symbols_exported():
    lib = cabi.library()
    declared = _declared_symbols()
    assert "oops_ta_forward" in declared and "oops_ta_backward" in declared
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in include/oops_ta.h but not exported"
    assert set(cabi.EXPORTS) <= set(declared)


def test_struct_layout_matches_header():
    # Pair: pointer + four int64 strides; Problem and Grads sizes follow from the field list in the header.
    assert ctypes.sizeof(cabi.Pair) == 40
    assert ctypes.sizeof(cabi.Problem) == 4 * 12 + 3 * 40 + 8 * 4 + 8 * 6 + 16
    assert ctypes.sizeof(cabi.Grads) == 3 * 40 + 8 * 6


def test_status_strings_and_version():
    lib = cabi.library()
    assert lib.oops_ta_abi_version() == cabi.ABI_VERSION
    assert lib.oops_ta_status_string(0) == b"ok"
    assert b"unknown" in lib.oops_ta_status_string(1234)


def _problem(**over):
    p = cabi.Problem()
    p.abi_version = cabi.ABI_VERSION
    p.dtype = cabi.BF16
    p.bias_dtype = cabi.BF16
    p.batch, p.rows, p.cols, p.heads, p.head_dim = 1, 8, 8, 2, 32
    p.scale = 1.0
    for key, value in over.items():
        setattr(p, key, value)
    return p


def test_admission_without_a_gpu():
    lib = cabi.library()
    assert lib.oops_ta_supported(ctypes.byref(_problem())) == 0
    assert lib.oops_ta_supported(ctypes.byref(_problem(head_dim=257))) == 3
    assert lib.oops_ta_supported(ctypes.byref(_problem(dtype=7))) == 2
    assert lib.oops_ta_supported(ctypes.byref(_problem(rows=0))) == 1
    assert lib.oops_ta_supported(ctypes.byref(_problem(abi_version=99))) == 1
    assert lib.oops_ta_supported(ctypes.byref(_problem(bias_groups=3))) == 1
    assert lib.oops_ta_supported(ctypes.byref(_problem(bias_groups=1, bias_dtype=cabi.F16))) == 2
    assert b"ABI" in lib.oops_ta_last_error() or lib.oops_ta_last_error() != b""
    assert lib.oops_ta_supported(None) == 1


def test_workspace_queries_are_host_only():
    lib = cabi.library()
    p = _problem(flags=cabi.FLAG_FORCE_GENERIC)
    assert lib.oops_ta_forward_workspace_bytes(ctypes.byref(p)) >= 1 * 8 * 2 * 8 * 8 * 4
    g = cabi.Grads()
    assert lib.oops_ta_backward_workspace_bytes(ctypes.byref(p), ctypes.byref(g)) > 0


def _tensor_problem(cols=100, bias_row=104, dtype=cabi.BF16, head_dim=32):
    p = _problem(dtype=dtype, bias_dtype=dtype, head_dim=head_dim)
    p.batch, p.rows, p.cols, p.heads = 1, cols, cols, 4
    for name in ("q", "k", "v"):
        pair = getattr(p, name)
        pair.ptr, pair.sh, pair.sc = 0x10000, head_dim, 4 * head_dim
        pair.sr, pair.sb = cols * 4 * head_dim, cols * cols * 4 * head_dim
    p.bias_groups, p.bias = 1, 0x20000
    p.bias_sk, p.bias_sq, p.bias_sh = 1, bias_row, cols * bias_row
    p.bias_sg = p.bias_sb = 4 * cols * bias_row
    return p


def test_kernel_selection_is_host_only():
    """Which kernel family serves a problem: tcgen05 for 16-bit, head_dim 32, 16-byte aligned rows."""
    lib = cabi.library()
    assert lib.oops_ta_uses_tensor_path(ctypes.byref(_tensor_problem()), 0) == 1
    assert lib.oops_ta_uses_tensor_path(ctypes.byref(_tensor_problem()), 1) == 1
    assert lib.oops_ta_uses_tensor_path(ctypes.byref(_tensor_problem(bias_row=100)), 0) == 0  # 200-byte rows
    assert lib.oops_ta_uses_tensor_path(ctypes.byref(_tensor_problem(head_dim=24)), 0) == 0
    assert lib.oops_ta_uses_tensor_path(ctypes.byref(_tensor_problem(dtype=cabi.F32)), 0) == 0
    forced = _tensor_problem()
    forced.flags = cabi.FLAG_FORCE_GENERIC
    assert lib.oops_ta_uses_tensor_path(ctypes.byref(forced), 0) == 0
