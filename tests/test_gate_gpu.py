"""GPU parity of the sigmoid gate: the reference-signature operator and the gate fused into triangle attention's
forward kernel, against the CPU oracles (reference: tests/attention/gate/test_gate_attention_output.py:40-43,
dense rows of its forward/backward matrix :150-240)."""

from __future__ import annotations

import pytest
import torch

import parity_bounds as parity
from oops_b200 import gate_attention_output, triangle_attention, triangle_attention_gated
from oracle import gate_oracle
from oracle import triangle_oracle as oracle

pytestmark = pytest.mark.gpu
ATOL = {torch.float32: 1e-4, torch.float16: 2e-2, torch.bfloat16: 3e-2}


def gate_case(dtype, shape, layout="head", seed=71):
    gen = torch.Generator().manual_seed(seed)
    *prefix, heads, length, head_size = shape
    channels, single_channels, out_channels = heads * head_size, 48, 31
    attention = torch.randn(shape, generator=gen)
    single = torch.randn(*prefix, length, single_channels, generator=gen)
    gate_weight = torch.randn(channels, single_channels, generator=gen) / single_channels**0.5
    output_weight = torch.randn(out_channels, channels, generator=gen) / 8
    upstream = torch.randn(*prefix, length, out_channels, generator=gen)
    return [t.to(dtype) for t in (attention, single, gate_weight, output_weight, upstream)], layout


@pytest.mark.parametrize(
    "dtype,shape,layout",
    [(torch.float32, (2, 4, 37, 16), "head"), (torch.float32, (4, 37, 16), "head"), (torch.float16, (2, 4, 57, 16), "head"),
     (torch.bfloat16, (2, 4, 449, 16), "token"), (torch.bfloat16, (2, 3, 4, 33, 32), "head"), (torch.float32, (2, 4, 37, 20), "negative")],
)
def test_gate_attention_output_forward_backward(cuda, dtype, shape, layout):
    (attention, single, gate_weight, output_weight, upstream), _ = gate_case(dtype, shape, layout)
    leaves = [t.to(cuda) for t in (attention, single, gate_weight, output_weight)]
    if layout == "token":  # token-major storage viewed head-major
        leaves[0] = leaves[0].transpose(-3, -2).contiguous().transpose(-3, -2)
    if layout == "negative":
        leaves = [-t for t in leaves]
    leaves = [t.detach().requires_grad_(True) for t in leaves]
    views = [torch._neg_view(t) for t in leaves] if layout == "negative" else leaves
    out = gate_attention_output(*views)
    grads = torch.autograd.grad(out, leaves, upstream.to(cuda))
    reference = [t.detach().clone().double().requires_grad_(True) for t in (attention, single, gate_weight, output_weight)]
    want = gate_oracle.gate_attention_output(*reference, compute_dtype=torch.float64)
    want_grads = torch.autograd.grad(want, reference, upstream.double())
    assert out.dtype == dtype and out.shape == want.shape
    atol = ATOL[dtype]
    tag = f"gate[{str(dtype).split('.')[-1]} {shape} {layout}]"
    parity.check(f"{tag} out", out, want, atol * max(1.0, float(want.abs().max())) if dtype is not torch.float32 else atol)
    sign = -1.0 if layout == "negative" else 1.0
    for name, got, ref in zip(("dattention", "dsingle", "dgate_weight", "doutput_weight"), grads, want_grads):
        assert got.shape == ref.shape and got.dtype == dtype
        parity.check(f"{tag} {name}", got, ref * sign, atol, relative_to_max=True)


@pytest.mark.parametrize(
    "dtype,n,dim,bias_kind,valid",
    [(torch.bfloat16, 200, 32, "shared", 170), (torch.float16, 136, 32, "none", None), (torch.float32, 40, 24, "shared", 33),
     (torch.bfloat16, 72, 16, "full", None)],
)
def test_gated_triangle_attention_against_the_oracles(cuda, dtype, n, dim, bias_kind, valid):
    """sigmoid(gate) * attention from the fused forward epilogue (tcgen05 kernels at head size 32, layout-agnostic
    kernels otherwise), and every gradient including the gate's, against the two oracles chained on the CPU."""
    gen = torch.Generator().manual_seed(13)
    heads, rows = 4, 9
    scale_in = 0.5 if dtype is not torch.float32 else 1.0
    q, k, v = ((torch.randn(1, rows, n, heads, dim, generator=gen) * scale_in).to(dtype) for _ in range(3))
    gate = torch.randn(1, rows, n, heads, dim, generator=gen).to(dtype)
    upstream = torch.randn(1, rows, n, heads, dim, generator=gen).to(dtype)
    bias = None
    if bias_kind != "none":
        bias = torch.randn(1, 1 if bias_kind == "shared" else rows, heads, n, n, generator=gen).to(dtype)
    mask = None
    if valid is not None:
        mask = (torch.arange(n) < valid)[None, None, :].expand(1, rows, n).contiguous()

    ref_leaves = [t.double().requires_grad_(True) for t in (q, k, v, gate)] + ([] if bias is None else [bias.double().requires_grad_(True)])
    attention = oracle.reference_dense(ref_leaves[0], ref_leaves[1], ref_leaves[2], mask, None if bias is None else ref_leaves[4],
                                       compute_dtype=torch.float64)
    want = gate_oracle.gated_values(attention, ref_leaves[3], compute_dtype=torch.float64)
    want_grads = torch.autograd.grad(want, ref_leaves, upstream.double())

    leaves = [t.to(cuda).requires_grad_(True) for t in (q, k, v, gate)] + ([] if bias is None else [bias.to(cuda).requires_grad_(True)])
    got = triangle_attention_gated(leaves[0], leaves[1], leaves[2], leaves[3], None if mask is None else mask.to(cuda),
                                   None if bias is None else leaves[4])
    grads = torch.autograd.grad(got, leaves, upstream.to(cuda))
    atol = 1e-4 if dtype is torch.float32 else 2e-2
    tag = f"gated[{str(dtype).split('.')[-1]} n={n} d={dim} bias={bias_kind}]"
    parity.check(f"{tag} out", got, want, atol)
    names = ("dq", "dk", "dv", "dgate") + (() if bias is None else ("dbias",))
    for name, g, w in zip(names, grads, want_grads):
        parity.check(f"{tag} {name}", g, w, atol, relative_to_max=dtype is not torch.float32)
    # inference takes the same kernel without the ungated copy, and equals the unfused composition bit for bit
    with torch.no_grad():
        fused = triangle_attention_gated(leaves[0], leaves[1], leaves[2], leaves[3], None if mask is None else mask.to(cuda),
                                         None if bias is None else leaves[4])
        plain = triangle_attention(leaves[0], leaves[1], leaves[2], None if mask is None else mask.to(cuda),
                                   None if bias is None else leaves[4])
    assert torch.equal(fused, got.detach())
    composed = (torch.sigmoid(leaves[3].detach().float()) * plain.float()).to(dtype)
    parity.check(f"{tag} fused vs composed", fused, composed.double(), 2.0 ** -7 * max(1.0, float(composed.abs().max())) if dtype is not torch.float32 else 1e-5)
