"""Parity of the benchmark configurations at their full sizes against the f32 oracle.

Every output and gradient the configurations name is compared with the oracle itself (not with another kernel of
this library): the whole tensor where the oracle finishes in seconds, a seeded sample of pair rows otherwise (rows
are independent softmax domains, so a row's out/dq/dk/dv do not depend on which other rows are present; the
shared-bias gradient is a sum over rows, so the operator is called on the sampled rows with the full bias and its
gradient compared with the oracle on the same rows).  Bounds are those of ``parity_bounds``.
"""

from __future__ import annotations

import pytest
import torch

import parity_bounds as parity
from oops_b200 import NestedTensor, triangle_attention
from oracle import triangle_oracle as oracle

pytestmark = pytest.mark.gpu

ATOL16 = 2e-2


def baseline_inputs(n, dtype, *, heads=4, dim=32, seed=0, scale_inputs=0.5):
    gen = torch.Generator().manual_seed(seed)
    q, k, v = ((torch.randn(1, n, n, heads, dim, generator=gen) * scale_inputs).to(dtype) for _ in range(3))
    bias = torch.randn(1, 1, heads, n, n, generator=gen).to(dtype)
    upstream = torch.randn(1, n, n, heads, dim, generator=gen).to(dtype)
    return q, k, v, bias, upstream


def run_operator(q, k, v, mask, bias, upstream, cuda):
    leaves = [t.to(cuda).detach().requires_grad_(True) for t in (q, k, v, bias)]
    out = triangle_attention(leaves[0], leaves[1], leaves[2], None if mask is None else mask.to(cuda), leaves[3])
    grads = torch.autograd.grad(out, leaves, upstream.to(cuda))
    return (out.detach(), *grads)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_config3_every_row_against_the_oracle(cuda, dtype):
    """Config 3 (starting node, N=768, H=4, D=32, forward+backward): out, dq, dk, dv and dbias of all 768 rows."""
    n = 768
    q, k, v, bias, upstream = baseline_inputs(n, dtype)
    mask = torch.ones(1, n, n, dtype=torch.bool)
    got = run_operator(q, k, v, mask, bias, upstream, cuda)
    want = oracle.forward_backward(q, k, v, mask, bias, upstream)
    tag = f"config3[{str(dtype).split('.')[-1]}]"
    for name, g, w in zip(("out", "dq", "dk", "dv"), got, want):
        parity.check(f"{tag} {name}", g, w, ATOL16)
    parity.check(f"{tag} dbias", got[4], want[4], ATOL16, relative_to_max=True)


def test_config5_sampled_rows_against_the_oracle(cuda):
    """Config 5 (N=2048): 96 seeded pair rows with the full 2048 x 2048 bias.  The call walks 16 key tiles, splits each
    row into groups of query tiles and sums the bias gradient over the sampled rows; all five results are compared
    with the oracle on the same rows."""
    n, sample = 2048, 96
    q, k, v, bias, upstream = baseline_inputs(n, torch.bfloat16, seed=11)
    rows = torch.randperm(n, generator=torch.Generator().manual_seed(2))[:sample].sort().values
    q, k, v, upstream = (t[:, rows].contiguous() for t in (q, k, v, upstream))
    mask = torch.ones(1, sample, n, dtype=torch.bool)
    got = run_operator(q, k, v, mask, bias, upstream, cuda)
    want = oracle.forward_backward(q, k, v, mask, bias, upstream)
    for name, g, w in zip(("out", "dq", "dk", "dv"), got, want):
        parity.check(f"config5[{sample} rows] {name}", g, w, ATOL16)
    parity.check(f"config5[{sample} rows] dbias", got[4], want[4], ATOL16, relative_to_max=True)


def test_config4_ending_node_ragged_with_token_masks(cuda):
    """Config 4 at its full lengths: ending-node ragged batch (1024 and 700 tokens), bf16, forward+backward, shared
    bias, per-sample token masks (the pair mask is the outer conjunction of a token mask with itself).

    The packed call is compared, bit for bit, with one dense ending-node call per sample (same kernels on the same
    strided views), and the dense calls are compared with the oracle: out/dq/dk/dv on a seeded sample of logical
    rows, and the bias gradient by running the operator on those rows alone."""
    lengths, heads, dim = (1024, 700), 4, 32
    gen = torch.Generator().manual_seed(6)
    dtype = torch.bfloat16
    stored = {name: [(torch.randn(L, L, heads, dim, generator=gen) * 0.5).to(dtype) for L in lengths] for name in "qkv"}
    biases = [torch.randn(1, heads, L, L, generator=gen).to(dtype) for L in lengths]
    tokens = [torch.rand(L, generator=gen) > 0.1 for L in lengths]
    for tok in tokens:
        tok[0] = True
    masks = [tok[:, None] & tok[None, :] for tok in tokens]
    ups = [torch.randn(L, L, heads, dim, generator=gen).to(dtype) for L in lengths]

    def packed(elements, ragged_dims):
        template = NestedTensor(elements, ragged_dims=ragged_dims)
        values = template.concat.to(cuda)
        return template, values

    leaves = {}
    nested = {}
    for name in "qkv":
        template, values = packed(stored[name], (0, 1))
        leaves[name] = values.detach().requires_grad_(True)
        nested[name] = template.packed_like(leaves[name]).transpose(-4, -3)
    mask_template, mask_values = packed(masks, (0, 1))
    nested_mask = mask_template.packed_like(mask_values).transpose(-2, -1)
    bias_template, bias_values = packed(biases, (2, 3))
    leaves["bias"] = bias_values.detach().requires_grad_(True)
    nested_bias = bias_template.packed_like(leaves["bias"]).transpose(-2, -1)
    up_template, up_values = packed(ups, (0, 1))

    out = triangle_attention(nested["q"], nested["k"], nested["v"], nested_mask, nested_bias).concat
    grads = torch.autograd.grad(out, [leaves[n] for n in ("q", "k", "v", "bias")], up_values)
    packed_results = dict(out=out.detach(), q=grads[0], k=grads[1], v=grads[2], bias=grads[3])

    cell_at, bias_at = 0, 0
    for i, L in enumerate(lengths):
        cells = L * L
        # the logical sample is the pair-axes transpose of the stored element (ending node); masks are symmetric
        logical = {name: stored[name][i].transpose(0, 1)[None] for name in "qkv"}
        logical_bias = biases[i].transpose(-2, -1)[None]
        logical_up = ups[i].transpose(0, 1)[None]
        mask = masks[i].t()[None]
        dense = run_operator(logical["q"], logical["k"], logical["v"], mask, logical_bias, logical_up, cuda)
        # packed results of this sample, in the stored order
        block = {name: packed_results[name][cell_at : cell_at + cells].reshape(L, L, heads, dim) for name in ("out", "q", "k", "v")}
        for name, dense_value in zip(("out", "q", "k", "v"), dense[:4]):
            assert torch.equal(block[name].transpose(0, 1), dense_value[0]), f"sample {i} {name}: packed and dense calls differ"
        packed_bias_grad = packed_results["bias"][bias_at : bias_at + cells].reshape(L, L, 1, heads).permute(2, 3, 0, 1)
        assert torch.equal(packed_bias_grad.transpose(-2, -1), dense[4][0]), f"sample {i}: packed and dense bias gradients differ"
        cell_at += cells
        bias_at += cells

        rows = torch.randperm(L, generator=torch.Generator().manual_seed(7 + i))[:48].sort().values
        rows = torch.cat([rows, torch.nonzero(~tokens[i])[:2, 0]]).unique()  # include rows of dropped tokens
        sub = lambda t: t[:, rows]  # noqa: E731
        want = oracle.forward_backward(sub(logical["q"]), sub(logical["k"]), sub(logical["v"]), sub(mask), logical_bias,
                                       sub(logical_up))
        tag = f"config4 sample {i} (N={L})"
        for name, g, w in zip(("out", "dq", "dk", "dv"), dense[:4], want[:4]):
            parity.check(f"{tag} {name}", g[:, rows], w, ATOL16)
        got_rows = run_operator(sub(logical["q"]), sub(logical["k"]), sub(logical["v"]), sub(mask), logical_bias,
                                sub(logical_up), cuda)
        parity.check(f"{tag} dbias[{len(rows)} rows]", got_rows[4], want[4], ATOL16, relative_to_max=True)
        # the rows of the sampled call are the same rows of the full call (row independence, same tiles)
        for name, g_rows, g_full in zip(("out", "dq", "dk", "dv"), got_rows[:4], dense[:4]):
            assert torch.equal(g_rows, g_full[:, rows]), f"{tag} {name}: a row's result depends on the other rows"


@pytest.mark.parametrize(
    "n,valid,bias_kind,swapped",
    [(296, 260, "shared", False), (200, 150, "none", False), (136, None, "full", False), (160, 131, "shared", True)],
)
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_head_size_32_tensor_kernels_against_the_oracle(cuda, dtype, n, valid, bias_kind, swapped):
    """Every 16-bit head-size-32 kernel (f16 and bf16 instantiations: forward, single-pass reverse, shared-bias and
    per-row bias gradients) on sizes with ragged last tiles, a padding mask and the ending-node memory form."""
    from oops_b200.runtime import cabi

    gen = torch.Generator().manual_seed(31)
    heads, dim = 4, 32
    q, k, v = ((torch.randn(1, n, n, heads, dim, generator=gen) * 0.5).to(dtype) for _ in range(3))
    upstream = torch.randn(1, n, n, heads, dim, generator=gen).to(dtype)
    bias = None
    if bias_kind != "none":
        bias = torch.randn(1, 1 if bias_kind == "shared" else n, heads, n, n, generator=gen).to(dtype)
    mask = None
    if valid is not None:
        tok = torch.arange(n) < valid
        mask = (tok[:, None] & tok[None, :])[None]
    want = oracle.forward_backward(q, k, v, mask, bias, upstream)

    def device_form(t):
        t = t.to(cuda)
        if swapped:  # pair axes exchanged in memory: the ending-node form, read through strides
            t = t.transpose(1, 2).contiguous().transpose(1, 2)
        return t.detach().requires_grad_(True)

    leaves = [device_form(t) for t in (q, k, v)]
    bias_leaf = None if bias is None else bias.to(cuda).requires_grad_(True)
    problem = cabi.make_problem(leaves[0].detach(), leaves[1].detach(), leaves[2].detach(), None,
                                None if bias_leaf is None else bias_leaf.detach(), dim**-0.5)
    assert cabi.library().oops_ta_uses_tensor_path(cabi.byref(problem), 1) == 1, "case must take the tcgen05 kernels"
    out = triangle_attention(leaves[0], leaves[1], leaves[2], None if mask is None else mask.to(cuda), bias_leaf)
    wanted = leaves + ([] if bias_leaf is None else [bias_leaf])
    grads = torch.autograd.grad(out, wanted, device_form(upstream).detach())
    tag = f"d32[{str(dtype).split('.')[-1]} n={n} valid={valid} bias={bias_kind}{' swapped' if swapped else ''}]"
    parity.check(f"{tag} out", out, want[0], ATOL16)
    for name, g, w in zip(("dq", "dk", "dv"), grads, want[1:4]):
        parity.check(f"{tag} {name}", g, w, ATOL16)
    if bias_leaf is not None:
        parity.check(f"{tag} dbias", grads[3], want[4], ATOL16, relative_to_max=bias_kind == "shared")
    if valid is not None:
        assert torch.count_nonzero(out[:, valid:]) == 0, "rows without a kept key must be exactly zero"
