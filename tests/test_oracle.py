"""The CPU oracle against the golden vectors produced by the reference's own `_reference`."""

from __future__ import annotations

from pathlib import Path

import pytest
import torch

from oracle import triangle_oracle as oracle

GOLDEN = Path(__file__).resolve().parent / "golden"
DENSE = ("dense_f32_shared_masked", "dense_f64_full_row0_empty", "dense_f32_plain", "dense_bf16_shared")


def _load(name):
    return torch.load(GOLDEN / f"{name}.pt", weights_only=False)


@pytest.mark.parametrize("name", DENSE)
@pytest.mark.parametrize("blocked", [False, True])
def test_dense_golden(name, blocked):
    g = _load(name)
    compute = torch.float64 if "float64" in g["compute_dtype"] else torch.float32
    budget = 1 if blocked else 1 << 30  # budget 1 byte forces one row per block
    out, dq, dk, dv, dbias = oracle.forward_backward(
        g["q"], g["k"], g["v"], g["mask"], g["bias"], g["upstream"], compute_dtype=compute, budget_bytes=budget
    )
    tol = dict(atol=1e-10, rtol=1e-10) if compute is torch.float64 else dict(atol=2e-6, rtol=1e-5)
    torch.testing.assert_close(out, g["out"], **tol)
    # the golden gradients were rounded to the f32 leaves' dtype by autograd
    tol = dict(atol=2e-6, rtol=1e-5) if g["dq"].dtype is torch.float32 else dict(atol=1e-2, rtol=8e-3)
    torch.testing.assert_close(dq, g["dq"].to(compute), **tol)
    torch.testing.assert_close(dk, g["dk"].to(compute), **tol)
    torch.testing.assert_close(dv, g["dv"].to(compute), **tol)
    if g["bias"] is not None:
        torch.testing.assert_close(dbias, g["dbias"].to(compute), **tol)
    fwd = oracle.forward(g["q"], g["k"], g["v"], g["mask"], g["bias"], compute_dtype=compute, budget_bytes=budget)
    torch.testing.assert_close(fwd, g["out"], **tol)


def test_fully_masked_row_is_zero():
    g = _load("dense_f64_full_row0_empty")
    out = oracle.forward(g["q"], g["k"], g["v"], g["mask"], g["bias"], compute_dtype=torch.float64)
    assert torch.count_nonzero(out[:, 0]) == 0
    assert torch.count_nonzero(g["out"][:, 0]) == 0


def test_config1_golden():
    g = _load("config1")
    gen = torch.Generator().manual_seed(g["seed"])
    n, h, d = g["n"], g["heads"], g["dim"]
    q, k, v = (torch.randn(1, n, n, h, d, generator=gen) for _ in range(3))
    bias = torch.randn(1, 1, h, n, n, generator=gen)
    upstream = torch.randn(1, n, n, h, d, generator=gen)
    checksum = torch.stack([t.double().sum() for t in (q, k, v, bias, upstream)])
    torch.testing.assert_close(checksum, g["input_checksum"], atol=1e-6, rtol=0)
    mask = torch.ones(1, n, n, dtype=torch.bool)
    out, dq, dk, dv, dbias = oracle.forward_backward(q, k, v, mask, bias, upstream, budget_bytes=1 << 20)
    tol = dict(atol=5e-6, rtol=1e-5)
    torch.testing.assert_close(out[:, ::4, ::4], g["out"], **tol)
    torch.testing.assert_close(dq[:, ::4, ::4], g["dq"], **tol)
    torch.testing.assert_close(dk[:, ::4, ::4], g["dk"], **tol)
    torch.testing.assert_close(dv[:, ::4, ::4], g["dv"], **tol)
    torch.testing.assert_close(dbias[..., ::2, ::2], g["dbias"], atol=2e-5, rtol=1e-5)


def test_nested_golden():
    g = _load("nested")
    parts = oracle.nested_forward(
        [e["q"] for e in g["elements"]], [e["k"] for e in g["elements"]], [e["v"] for e in g["elements"]],
        [e["mask"] for e in g["elements"]], [e["bias"] for e in g["elements"]],
    )
    torch.testing.assert_close(oracle.flatten_nested(parts), g["packed"], atol=2e-6, rtol=1e-5)
    torch.testing.assert_close(
        oracle.flatten_nested(parts, transposed_pair_axes=True), g["packed_transposed"], atol=2e-6, rtol=1e-5
    )


def test_flops_formula():
    assert oracle.flops(1, 768, 768, 4, 32, backward=True) == pytest.approx(8.117e11, rel=1e-3)
    assert oracle.flops(1, 2048, 2048, 4, 32, backward=False) == pytest.approx(4.398e12, rel=1e-3)


@pytest.mark.parametrize("name", ["f32_rank4", "f64_rank3", "f32_rank5"])
def test_gate_oracle_matches_the_reference_statement(name):
    """The gate oracle against outputs and autograd gradients of the reference's own `_reference`
    (tests/attention/gate/test_gate_attention_output.py:40-43), stored in tests/golden/gate.pt."""
    from oracle import gate_oracle

    case = torch.load(GOLDEN / "gate.pt", weights_only=False)[name]
    dtype = case["attention"].dtype
    leaves = [case[n].clone().requires_grad_(True) for n in ("attention", "single", "gate_weight", "output_weight")]
    out = gate_oracle.gate_attention_output(*leaves, compute_dtype=dtype)
    tol = dict(atol=1e-10, rtol=1e-10) if dtype is torch.float64 else dict(atol=2e-6, rtol=1e-5)
    torch.testing.assert_close(out, case["out"], **tol)
    for got, want in zip(torch.autograd.grad(out, leaves, case["upstream"]), case["grads"]):
        torch.testing.assert_close(got, want, **tol)
    # the element-wise core alone, in the token-major layout the fused epilogue works in
    attention, single, gate_weight, output_weight = (case[n] for n in ("attention", "single", "gate_weight", "output_weight"))
    *prefix, heads, length, head_size = attention.shape
    token_major = attention.transpose(-3, -2).reshape(*prefix, length, heads * head_size)
    gated = gate_oracle.gated_values(token_major, torch.nn.functional.linear(single, gate_weight), compute_dtype=dtype)
    torch.testing.assert_close(torch.nn.functional.linear(gated, output_weight), case["out"], **tol)
