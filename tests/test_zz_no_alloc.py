"""The allocation-free forward entry point (`oops_ta_forward_static`) against the regular one.

This entry point exists for hosts that must not allocate device memory when they call -- a server whose
memory pool is frozen after start-up, a latency-critical loop that cannot afford the device-wide
synchronisation of an allocation, or code that is recording work for later replay.  It keeps the logits of
a block of pair rows in a fixed array inside the library instead of a caller-provided workspace.

The test drives it through the C ABI several times in a row (the array keeps the previous call's contents) and
compares each result with `oops_ta_forward` on the same kernels (layout-agnostic path forced), which must
agree bit for bit, and with the CPU oracle within the tolerance of the dtype.  One case has more pair rows than
the array holds at once, so the entry point walks the rows in blocks that reuse the array within a single call
(the regular call splits by its own, larger budget: equal bits also show that results do not depend on the block
size).  A problem whose single pair row does not fit is refused.
This file is named so that pytest collects it last.
"""

from __future__ import annotations

import pytest
import torch

from oracle import triangle_oracle as oracle

pytestmark = pytest.mark.gpu
ATOL = {torch.float32: 1e-4, torch.bfloat16: 2e-2}


def _case(cuda, seed, rows, cols, heads, dim, dtype):
    gen = torch.Generator().manual_seed(seed)
    q, k, v = (torch.randn(1, rows, cols, heads, dim, generator=gen).to(dtype).to(cuda) for _ in range(3))
    bias = torch.randn(1, 1, heads, cols, cols, generator=gen).to(dtype).to(cuda)
    mask = (torch.rand(1, rows, cols, generator=gen) > 0.2).to(cuda)
    mask[..., 0] = True
    return q, k, v, mask, bias


def _regular(lib, cabi, q, k, v, mask, bias, scale, stream):
    problem = cabi.make_problem(q, k, v, mask, bias, scale, cabi.FLAG_FORCE_GENERIC)
    scratch = torch.empty(int(lib.oops_ta_forward_workspace_bytes(cabi.byref(problem))) + 1, dtype=torch.uint8, device=q.device)
    problem.workspace, problem.workspace_bytes = scratch.data_ptr(), scratch.numel()
    out = torch.empty_like(q)
    lse = torch.empty(q.shape[0] * q.shape[1] * q.shape[3] * q.shape[2], dtype=torch.float32, device=q.device)
    pair = cabi.pair_of(out)
    assert lib.oops_ta_forward(cabi.byref(problem), cabi.byref(pair), lse.data_ptr(), stream) == 0
    return out, lse


def _static(lib, cabi, q, k, v, mask, bias, scale, stream):
    problem = cabi.make_problem(q, k, v, mask, bias, scale)  # no workspace is attached
    out = torch.empty_like(q)
    lse = torch.empty(q.shape[0] * q.shape[1] * q.shape[3] * q.shape[2], dtype=torch.float32, device=q.device)
    pair = cabi.pair_of(out)
    status = lib.oops_ta_forward_static(cabi.byref(problem), cabi.byref(pair), lse.data_ptr(), stream)
    assert status == 0, cabi.status_message(status)
    return out, lse


def test_static_forward_matches_regular_forward_twice(cuda):
    from oops_b200.runtime import cabi

    lib = cabi.library()
    stream = torch.cuda.current_stream().cuda_stream
    assert lib.oops_ta_forward_static_capacity() == 32 << 20
    # calls in a row with different shapes and dtypes: each sees the previous one's leftovers in the array.  The last
    # case needs 4 MiB of logits per pair row (4 heads x 512^2 x 4 bytes), so its 16 rows take two blocks of 8.
    cases = ((0, 5, 70, 2, 24, torch.float32), (1, 9, 130, 4, 32, torch.bfloat16), (2, 16, 512, 4, 16, torch.bfloat16))
    for seed, rows, cols, heads, dim, dtype in cases:
        q, k, v, mask, bias = _case(cuda, seed, rows, cols, heads, dim, dtype)
        scale = dim**-0.5
        want_out, want_lse = _regular(lib, cabi, q, k, v, mask, bias, scale, stream)
        got_out, got_lse = _static(lib, cabi, q, k, v, mask, bias, scale, stream)
        torch.cuda.synchronize()
        assert torch.equal(got_out, want_out)
        assert torch.equal(got_lse, want_lse)
        reference = oracle.forward(q.cpu(), k.cpu(), v.cpu(), mask.cpu(), bias.cpu(), scale)
        error = float((got_out.float().cpu() - reference).abs().max())
        assert error <= ATOL[dtype], f"rows={rows} cols={cols} {dtype}: max-abs error {error:.3e} against the oracle"


def test_static_forward_refuses_oversized_rows(cuda):
    from oops_b200.runtime import cabi

    lib = cabi.library()
    # one pair row needs heads * cols^2 * 4 bytes = 4 * 1536^2 * 4 = 36 MiB > 32 MiB; nothing is dereferenced
    cols, heads = 1536, 4
    q = torch.empty(1, 1, cols, heads, 8, dtype=torch.bfloat16, device=cuda)
    problem = cabi.make_problem(q, q, q, None, None, 1.0)
    out = torch.empty_like(q)
    pair = cabi.pair_of(out)
    status = lib.oops_ta_forward_static(cabi.byref(problem), cabi.byref(pair), None, torch.cuda.current_stream().cuda_stream)
    assert status == 5  # OOPS_TA_LIMIT_EXCEEDED
    assert "built-in scratch" in cabi.status_message(status)
