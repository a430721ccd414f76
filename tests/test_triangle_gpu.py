"""GPU parity of triangle attention against the CPU oracle and the golden vectors.

The matrix follows the reference's own test file
(tests/attention/triangle/test_triangle_attention.py: test_forward :226-258,
test_backward :260-419, test_contract :421-581), re-expressed for this package,
with the stricter tolerances of the build target: f32 <= 1e-4 and bf16/f16 <= 2e-2
max-abs against an f32 (or f64) oracle.
"""

from __future__ import annotations

from pathlib import Path

import pytest
import torch

from oops_b200 import NestedTensor, triangle_attention
from oops_b200.attention.triangle.triangle_attention import layout_agnostic_kernels, separate_reverse_kernels
from oracle import triangle_oracle as oracle

pytestmark = pytest.mark.gpu

GOLDEN = Path(__file__).resolve().parent / "golden"
ATOL = {torch.float32: 1e-4, torch.float16: 2e-2, torch.bfloat16: 2e-2}


def max_abs(a, b):
    return float((a.double().cpu() - b.double().cpu()).abs().max())


def assert_within(actual, expected, atol, what=""):
    assert actual.shape == expected.shape, (what, actual.shape, expected.shape)
    err = max_abs(actual, expected)
    assert err <= atol, f"{what}: max-abs error {err:.3e} > {atol:.1e}"


# ------------------------------------------------------------------------------------------
# dense cases
# ------------------------------------------------------------------------------------------


def dense_case(dtype, *, prefix=(2,), rows=4, cols=33, heads=2, dim=24, bias_kind="shared", mask_kind="random",
               swapped=False, negative=False, seed=0, scale_inputs=1.0):
    gen = torch.Generator().manual_seed(seed)
    shape = (*prefix, rows, cols, heads, dim)
    q, k, v = ((torch.randn(shape, generator=gen) * scale_inputs).to(dtype) for _ in range(3))
    bias = None
    if bias_kind != "none":
        groups = 1 if bias_kind == "shared" else rows
        bias = torch.randn((*prefix, groups, heads, cols, cols), generator=gen).to(dtype)
    mask = None
    if mask_kind != "none":
        mask = torch.rand((*prefix, rows, cols), generator=gen) > 0.2
        mask[..., 0] = True
        if mask_kind == "row0_empty":
            mask[..., 0, :] = False
    upstream = torch.randn(shape, generator=gen).to(dtype)
    return dict(q=q, k=k, v=v, mask=mask, bias=bias, upstream=upstream, swapped=swapped, negative=negative)


def to_device(case, cuda, active=("q", "k", "v", "bias")):
    """Move a case to the GPU in the requested memory form and mark the differentiable leaves."""
    leaves, args = {}, {}
    for name in ("q", "k", "v", "bias"):
        t = case[name]
        if t is None:
            args[name] = None
            continue
        t = t.to(cuda)
        if case["negative"]:
            t = -t  # the leaf holds the negated data; the operator sees a lazy-negation view of it
        if case["swapped"] and name != "bias":
            t = t.transpose(-4, -3).contiguous()
        t = t.detach().requires_grad_(name in active)
        leaves[name] = t
        view = t
        if case["swapped"] and name != "bias":
            view = view.transpose(-4, -3)
        if case["negative"]:
            view = torch._neg_view(view)
        args[name] = view
    args["mask"] = None if case["mask"] is None else case["mask"].to(cuda)
    return args, leaves


def oracle_dense(case, compute_dtype=torch.float32):
    q, k, v, mask, bias, up = (case[n] for n in ("q", "k", "v", "mask", "bias", "upstream"))
    flat = lambda t, tail: None if t is None else t.reshape(-1, *t.shape[-tail:])  # noqa: E731
    out, dq, dk, dv, db = oracle.forward_backward(
        flat(q, 4), flat(k, 4), flat(v, 4), None if mask is None else mask.reshape(-1, *mask.shape[-2:]),
        flat(bias, 4), flat(up, 4), compute_dtype=compute_dtype,
    )
    shape = q.shape
    return (out.reshape(shape), dq.reshape(shape), dk.reshape(shape), dv.reshape(shape),
            None if db is None else db.reshape(bias.shape))


def run_dense(case, cuda, active=("q", "k", "v", "bias"), atol=None, compute_dtype=torch.float32):
    dtype = case["q"].dtype
    atol = ATOL[dtype] if atol is None else atol
    args, leaves = to_device(case, cuda, active)
    out = triangle_attention(args["q"], args["k"], args["v"], args["mask"], args["bias"])
    want_out, want_dq, want_dk, want_dv, want_db = oracle_dense(case, compute_dtype)
    assert out.dtype == dtype and out.shape == case["q"].shape
    assert_within(out, want_out, atol, "out")
    wanted = [leaves[n] for n in ("q", "k", "v", "bias") if n in leaves and leaves[n].requires_grad]
    if not wanted:
        return out
    upstream = case["upstream"].to(cuda)
    grads = torch.autograd.grad(out, wanted, upstream)
    sign = -1.0 if case["negative"] else 1.0
    expected = dict(q=want_dq, k=want_dk, v=want_dv, bias=want_db)
    names = [n for n in ("q", "k", "v", "bias") if n in leaves and leaves[n].requires_grad]
    for name, grad, leaf in zip(names, grads, wanted):
        assert grad.dtype == leaf.dtype and grad.shape == leaf.shape
        want = expected[name] * sign
        if case["swapped"] and name != "bias":
            want = want.transpose(-4, -3)
        # gradients scale with the upstream magnitude; bf16 leaves round at ~2^-9 relative
        scale = 1.0 if dtype is torch.float32 else max(1.0, float(want.abs().max()))
        assert_within(grad, want, atol * scale, f"d{name}")
    return out


@pytest.mark.parametrize(
    "dtype,kwargs",
    [
        (torch.float32, dict(bias_kind="none")),
        (torch.float32, dict(bias_kind="full", negative=True)),
        (torch.float16, dict(bias_kind="shared", swapped=True)),
        (torch.bfloat16, dict(bias_kind="full", prefix=(2, 3))),
        (torch.float32, dict(bias_kind="full")),
        (torch.bfloat16, dict(bias_kind="shared", cols=41, dim=16)),
        (torch.float32, dict(bias_kind="shared", prefix=(), rows=3)),
    ],
)
def test_forward_dense(cuda, dtype, kwargs):
    case = dense_case(dtype, **kwargs)
    with torch.no_grad():
        run_dense(case, cuda, active=())


@pytest.mark.parametrize(
    "dtype,kwargs,active",
    [
        (torch.float32, dict(rows=17, cols=17, dim=129, bias_kind="shared", mask_kind="row0_empty", seed=117), ("q", "k", "v", "bias")),
        (torch.float32, dict(rows=17, cols=17, dim=129, bias_kind="shared", mask_kind="row0_empty", negative=True), ("q", "k", "v", "bias")),
        (torch.float32, dict(rows=17, cols=17, dim=129, bias_kind="none", mask_kind="row0_empty"), ("q", "k", "v")),
        (torch.float32, dict(rows=17, cols=17, dim=137, bias_kind="full", mask_kind="row0_empty"), ("q",)),
        (torch.float32, dict(rows=17, cols=17, dim=129, bias_kind="shared", mask_kind="row0_empty"), ("k",)),
        (torch.float32, dict(rows=17, cols=17, dim=137, bias_kind="full", mask_kind="row0_empty", swapped=True), ("bias",)),
        (torch.float32, dict(rows=17, cols=17, dim=255, bias_kind="shared", mask_kind="row0_empty", prefix=(2, 3)), ("v",)),
        (torch.float32, dict(dim=32, bias_kind="shared"), ("q", "k", "v", "bias")),
        (torch.bfloat16, dict(dim=32, bias_kind="full", swapped=True), ("q", "k", "v", "bias")),
        (torch.float32, dict(dim=24, bias_kind="full"), ("q", "k", "v", "bias")),
        (torch.float32, dict(dim=24, bias_kind="full", negative=True), ("q", "k", "v", "bias")),
        (torch.float16, dict(dim=24, bias_kind="shared", swapped=True), ("q",)),
        (torch.bfloat16, dict(dim=24, bias_kind="none", prefix=(2, 3)), ("k",)),
        (torch.bfloat16, dict(dim=16, cols=19, bias_kind="shared"), ("q", "k", "v", "bias")),
        (torch.float32, dict(dim=128, bias_kind="shared"), ("bias",)),
        (torch.float16, dict(dim=129, bias_kind="shared"), ("bias",)),
    ],
)
def test_backward_dense(cuda, dtype, kwargs, active):
    compute = torch.float64 if kwargs.get("dim", 0) > 128 else torch.float32
    run_dense(dense_case(dtype, **kwargs), cuda, active=active, compute_dtype=compute)


def test_sum_upstream_and_saved_strided_hook(cuda):
    """Gradients with an expanded (stride-0) upstream and with saved tensors that come back re-strided."""
    case = dense_case(torch.float32, dim=24, bias_kind="shared")
    args, leaves = to_device(case, cuda)

    def unpack(value):
        storage = value.new_empty(value.numel() * 2)
        view = storage[::2].reshape(value.shape)
        view.copy_(value)
        return view

    with torch.autograd.graph.saved_tensors_hooks(lambda value: value.detach(), unpack):
        out = triangle_attention(args["q"], args["k"], args["v"], args["mask"], args["bias"])
    out.sum().backward()
    case["upstream"] = torch.ones_like(case["upstream"])
    _, dq, dk, dv, db = oracle_dense(case)
    for name, want in (("q", dq), ("k", dk), ("v", dv), ("bias", db)):
        assert_within(leaves[name].grad, want, 1e-4, f"d{name}")


def test_inference_then_training_and_checkpoint(cuda):
    from torch.utils.checkpoint import checkpoint

    case = dense_case(torch.bfloat16, dim=16, cols=19, bias_kind="shared")
    args, leaves = to_device(case, cuda)
    with torch.inference_mode():
        triangle_attention(args["q"], args["k"], args["v"], args["mask"], args["bias"])
    out = checkpoint(triangle_attention, args["q"], args["k"], args["v"], args["mask"], args["bias"],
                     use_reentrant=False)
    grads = torch.autograd.grad(out, [leaves[n] for n in ("q", "k", "v", "bias")], case["upstream"].to(cuda))
    _, dq, dk, dv, db = oracle_dense(case)
    for grad, want in zip(grads, (dq, dk, dv, db)):
        assert_within(grad, want, 2e-2 * max(1.0, float(want.abs().max())))


def test_masked_nonfinite_is_exact_zero(cuda):
    q, k, v = (torch.full((1, 17, 17, 2, 129), float("inf"), device=cuda, requires_grad=True) for _ in range(3))
    mask = torch.zeros(1, 17, 17, device=cuda, dtype=torch.bool)
    bias = torch.full((1, 1, 2, 17, 17), float("nan"), device=cuda, requires_grad=True)
    out = triangle_attention(q, k, v, mask, bias)
    assert torch.count_nonzero(out) == 0 and not torch.isnan(out).any()
    for grad in torch.autograd.grad(out.sum(), (q, k, v, bias)):
        assert torch.count_nonzero(grad) == 0 and not torch.isnan(grad).any()


@pytest.mark.parametrize("dtype,dim", [(torch.bfloat16, 32), (torch.float32, 24)])
def test_masked_nonfinite_partial(cuda, dtype, dim):
    """Non-finite key/value rows behind the mask must not leak (reference kernel.py:220-223)."""
    case = dense_case(dtype, dim=dim, cols=40, bias_kind="shared")
    dropped = ~case["mask"]
    poisoned = {n: case[n].clone() for n in ("k", "v")}
    for n in ("k", "v"):
        poisoned[n][dropped] = float("inf")
    args, leaves = to_device({**case, **poisoned}, cuda)
    out = triangle_attention(args["q"], args["k"], args["v"], args["mask"], args["bias"])
    want = oracle_dense(case)
    assert_within(out, want[0], ATOL[dtype], "out")
    grads = torch.autograd.grad(out, [leaves[n] for n in ("q", "k", "v", "bias")], case["upstream"].to(cuda))
    for name, grad, ref in zip(("q", "k", "v", "bias"), grads, want[1:]):
        assert torch.isfinite(grad).all(), name
        assert_within(grad, ref, ATOL[dtype] * max(1.0, float(ref.abs().max())), f"d{name}")


def test_alias_and_determinism(cuda):
    case = dense_case(torch.float32, dim=24, bias_kind="shared")
    q = case["q"].to(cuda).requires_grad_(True)
    bias = case["bias"].to(cuda).requires_grad_(True)
    mask = case["mask"].to(cuda)
    results = []
    for _ in range(2):
        out = triangle_attention(q, q, q, mask, bias)
        results.append((out, *torch.autograd.grad(out, (q, bias), case["upstream"].to(cuda))))
    for first, second in zip(*results):
        assert torch.equal(first, second)
    aliased = {**case, "k": case["q"], "v": case["q"]}
    want_out, dq, dk, dv, db = oracle_dense(aliased)
    assert_within(results[0][0], want_out, 1e-4)
    assert_within(results[0][1], dq + dk + dv, 3e-4)
    assert_within(results[0][2], db, 1e-4)


def test_cuda_graph_replay(cuda):
    case = dense_case(torch.float32, dim=24, bias_kind="shared")
    args, _ = to_device(case, cuda, active=())
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.no_grad(), torch.cuda.stream(stream):
        for _ in range(3):
            triangle_attention(args["q"], args["k"], args["v"], args["mask"], args["bias"])
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            out = triangle_attention(args["q"], args["k"], args["v"], args["mask"], args["bias"])
        args["q"].add_(0.1)
        graph.replay()
    stream.synchronize()
    case["q"] = case["q"] + 0.1
    assert_within(out, oracle_dense(case)[0], 1e-4)


# ------------------------------------------------------------------------------------------
# golden vectors through the GPU path
# ------------------------------------------------------------------------------------------


@pytest.mark.parametrize("name", ["dense_f32_shared_masked", "dense_f64_full_row0_empty", "dense_f32_plain",
                                  "dense_bf16_shared"])
def test_golden_dense(cuda, name):
    g = torch.load(GOLDEN / f"{name}.pt", weights_only=False)
    dtype = g["q"].dtype
    leaves = [g[n].to(cuda).requires_grad_(True) for n in ("q", "k", "v")]
    bias = None if g["bias"] is None else g["bias"].to(cuda).requires_grad_(True)
    mask = None if g["mask"] is None else g["mask"].to(cuda)
    out = triangle_attention(*leaves, mask, bias)
    atol = ATOL[dtype]
    assert_within(out, g["out"], atol, "out")
    wanted = leaves + ([] if bias is None else [bias])
    grads = torch.autograd.grad(out, wanted, g["upstream"].to(cuda).to(dtype))
    for name_, grad in zip(("dq", "dk", "dv", "dbias"), grads):
        want = g[name_]
        assert_within(grad, want, atol * max(1.0, float(want.abs().max())), name_)


def test_golden_config1(cuda):
    """BASELINE config 1: f32, B=1, N=64, H=4, D=32, shared bias, all-ones mask, seed 0; <= 1e-4."""
    g = torch.load(GOLDEN / "config1.pt", weights_only=False)
    gen = torch.Generator().manual_seed(g["seed"])
    n, h, d = g["n"], g["heads"], g["dim"]
    q, k, v = (torch.randn(1, n, n, h, d, generator=gen) for _ in range(3))
    bias = torch.randn(1, 1, h, n, n, generator=gen)
    upstream = torch.randn(1, n, n, h, d, generator=gen)
    leaves = [t.to(cuda).requires_grad_(True) for t in (q, k, v, bias)]
    mask = torch.ones(1, n, n, dtype=torch.bool, device=cuda)
    out = triangle_attention(leaves[0], leaves[1], leaves[2], mask, leaves[3], scale=d**-0.5)
    assert_within(out[:, ::4, ::4], g["out"], 1e-4, "out")
    dq, dk, dv, db = torch.autograd.grad(out, leaves, upstream.to(cuda))
    assert_within(dq[:, ::4, ::4], g["dq"], 1e-4, "dq")
    assert_within(dk[:, ::4, ::4], g["dk"], 1e-4, "dk")
    assert_within(dv[:, ::4, ::4], g["dv"], 1e-4, "dv")
    assert_within(db[..., ::2, ::2], g["dbias"], 2e-4, "dbias")  # sums 64 rows of magnitude-~1 terms


# ------------------------------------------------------------------------------------------
# ragged (NestedTensor) cases
# ------------------------------------------------------------------------------------------


def nested_case(dtype, cuda, *, lengths=(3, 5), heads=2, dim=16, bias_kind="shared", with_mask=True, prefix=(),
                broadcast_prefix=False, transposed=False, seed=0):
    gen = torch.Generator().manual_seed(seed)
    rank = len(prefix)
    elements = {n: [torch.randn(*prefix, L, L, heads, dim, generator=gen).to(dtype) for L in lengths] for n in "qkv"}
    masks = None
    if with_mask:
        mask_prefix = (1,) * rank if broadcast_prefix else prefix
        masks = []
        for L in lengths:
            m = torch.rand(*mask_prefix, L, L, generator=gen) > 0.2
            m[..., 0] = True
            masks.append(m.expand(*prefix, L, L))
    biases, groups = None, None
    if bias_kind != "none":
        bias_prefix = (1,) * rank if broadcast_prefix else prefix
        groups = [1 if bias_kind == "shared" or (bias_kind == "mixed" and i == 0) else L
                  for i, L in enumerate(lengths)]
        biases = [torch.randn(*bias_prefix, g, heads, L, L, generator=gen).to(dtype) for g, L in zip(groups, lengths)]
    return dict(elements=elements, masks=masks, biases=biases, lengths=lengths, prefix=prefix, transposed=transposed,
                bias_kind=bias_kind, rank=rank)


def build_nested(case, cuda, requires_grad=True):
    rank = case["rank"]
    out = {}
    leaves = {}
    for n in "qkv":
        template = NestedTensor(case["elements"][n], ragged_dims=(rank, rank + 1))
        values = template.concat.to(cuda).detach().requires_grad_(requires_grad)
        leaves[n] = values
        nested = template.packed_like(values)
        out[n] = nested.transpose(-4, -3) if case["transposed"] else nested
    # With transposed q/k/v the *logical* sample is the transpose of the stored element.
    mask = None
    if case["masks"] is not None:
        template = NestedTensor([m.contiguous() for m in case["masks"]], ragged_dims=(rank, rank + 1))
        mask = template.packed_like(template.concat.to(cuda))
        if case["transposed"]:
            mask = mask.transpose(-2, -1)
    bias = None
    if case["biases"] is not None:
        if case["bias_kind"] == "shared":
            template = NestedTensor(case["biases"], ragged_dims=(rank + 2, rank + 3))
        else:
            template = NestedTensor(case["biases"], ragged_dims=(rank, rank + 2, rank + 3))
        values = template.concat.to(cuda).detach().requires_grad_(requires_grad)
        leaves["bias"] = values
        bias = template.packed_like(values)
        if case["transposed"]:
            bias = bias.transpose(-2, -1)
    return out["q"], out["k"], out["v"], mask, bias, leaves


def nested_oracle(case, upstream_packed, compute_dtype=torch.float32):
    """Per-sample oracle on the logical samples; returns packed out and packed grads for q, k, v, bias."""
    t = case["transposed"]
    rank = case["rank"]
    pa, pb = rank, rank + 1
    outs, grads = [], {n: [] for n in ("q", "k", "v", "bias")}
    at = 0
    for i, L in enumerate(case["lengths"]):
        logical = {n: (case["elements"][n][i].transpose(pa, pb) if t else case["elements"][n][i]) for n in "qkv"}
        mask = None if case["masks"] is None else case["masks"][i]
        if mask is not None and t:
            mask = mask.transpose(-2, -1)
        bias = None if case["biases"] is None else case["biases"][i]
        if bias is not None:
            bias = bias.transpose(-2, -1) if t else bias
            bias = bias.expand(*case["prefix"], *bias.shape[rank:])
        cells = L * L
        up = upstream_packed[at : at + cells].cpu()
        at += cells
        # packed order of the sample's output: (first pair axis, second, *prefix, H, D) of the *stored* element
        up = up.reshape(L, L, *up.shape[1:])
        order = (*range(2, 2 + rank), 0, 1, 2 + rank, 3 + rank)
        up_stored = up.permute(order)
        up_logical = up_stored.transpose(pa, pb) if t else up_stored
        flat = lambda x, tail: x.reshape(-1, *x.shape[-tail:])  # noqa: E731
        o, dq, dk, dv, db = oracle.forward_backward(
            flat(logical["q"], 4), flat(logical["k"], 4), flat(logical["v"], 4),
            None if mask is None else mask.reshape(-1, L, L), None if bias is None else flat(bias, 4),
            flat(up_logical, 4), compute_dtype=compute_dtype,
        )
        shape = logical["q"].shape

        def stored(x):
            x = x.reshape(shape)
            return x.transpose(pa, pb) if t else x

        outs.append(stored(o))
        for n, g in (("q", dq), ("k", dk), ("v", dv)):
            grads[n].append(stored(g))
        if db is not None:
            db = db.reshape(*case["prefix"], *db.shape[1:])
            own = case["biases"][i]
            # sum over broadcast prefix axes, back to the stored orientation
            for axis in range(rank):
                if own.shape[axis] == 1 and db.shape[axis] != 1:
                    db = db.sum(axis, keepdim=True)
            grads["bias"].append(db.transpose(-2, -1) if t else db)
    packed_out = oracle.flatten_nested(outs)
    packed = {n: oracle.flatten_nested(grads[n]) for n in "qkv"}
    if grads["bias"]:
        if case["bias_kind"] == "shared":
            template = NestedTensor(grads["bias"], ragged_dims=(rank + 2, rank + 3))
        else:
            template = NestedTensor(grads["bias"], ragged_dims=(rank, rank + 2, rank + 3))
        packed["bias"] = template.concat
    return packed_out, packed


@pytest.mark.parametrize(
    "dtype,kwargs",
    [
        (torch.float32, dict(bias_kind="shared")),
        (torch.bfloat16, dict(bias_kind="mixed")),
        (torch.float32, dict(bias_kind="full", transposed=True)),
        (torch.bfloat16, dict(bias_kind="mixed", prefix=(2, 3), broadcast_prefix=True)),
        (torch.float32, dict(bias_kind="shared", prefix=(2, 3), broadcast_prefix=True, transposed=True)),
        (torch.float32, dict(bias_kind="shared", lengths=(17, 19), dim=129)),
        (torch.float32, dict(bias_kind="mixed", lengths=(17, 19), dim=137, transposed=True)),
        (torch.float32, dict(bias_kind="none", with_mask=False, lengths=(7, 11), dim=24)),
        (torch.bfloat16, dict(bias_kind="shared", lengths=(40, 33), heads=4, dim=32, transposed=True)),
    ],
)
def test_nested(cuda, dtype, kwargs):
    case = nested_case(dtype, cuda, **kwargs)
    q, k, v, mask, bias, leaves = build_nested(case, cuda)
    out = triangle_attention(q, k, v, mask, bias)
    assert out.ragged_dims == q.ragged_dims and out.packed_dim_order == q.packed_dim_order
    values = out.concat
    gen = torch.Generator().manual_seed(9)
    upstream = torch.randn(values.shape, generator=gen).to(dtype)
    compute = torch.float64 if kwargs.get("dim", 16) > 128 else torch.float32
    want_out, want = nested_oracle(case, upstream, compute)
    atol = ATOL[dtype]
    assert_within(values, want_out, atol, "out")
    names = [n for n in ("q", "k", "v", "bias") if n in leaves]
    grads = torch.autograd.grad(values, [leaves[n] for n in names], upstream.to(cuda))
    for name, grad in zip(names, grads):
        assert grad.shape == leaves[name].shape and grad.dtype == dtype
        assert_within(grad, want[name], atol * max(1.0, float(want[name].abs().max())), f"d{name}")


# ----------------------------------------------------------------------------------------------
# torch.compile and FakeTensorMode (reference: test_triangle_attention.py:225-256 "compile" rows, :556-565 "fake")
# ----------------------------------------------------------------------------------------------


@pytest.mark.parametrize("dtype,prefix,bias_kind", [(torch.bfloat16, (2, 2), "full"), (torch.float32, (2,), "shared")])
def test_compiled_dense(cuda, dtype, prefix, bias_kind):
    torch._dynamo.reset()
    execute = torch.compile(lambda *inputs: triangle_attention(*inputs), fullgraph=True, dynamic=True)
    for cols in (33, 41):
        case = dense_case(dtype, prefix=prefix, cols=cols, bias_kind=bias_kind)
        args, leaves = to_device(case, cuda)
        out = execute(args["q"], args["k"], args["v"], args["mask"], args["bias"])
        want_out, want_dq, want_dk, want_dv, want_db = oracle_dense(case)
        assert out.dtype == dtype and out.shape == case["q"].shape
        assert_within(out, want_out, ATOL[dtype], f"out cols={cols}")
        grads = torch.autograd.grad(out, [leaves[n] for n in ("q", "k", "v", "bias")], case["upstream"].to(cuda))
        for name, grad, want in zip(("q", "k", "v", "bias"), grads, (want_dq, want_dk, want_dv, want_db)):
            scale = 1.0 if dtype is torch.float32 else max(1.0, float(want.abs().max()))
            assert_within(grad, want, ATOL[dtype] * scale, f"d{name} cols={cols}")


def test_compiled_nested(cuda):
    torch._dynamo.reset()

    def run(*inputs):
        return triangle_attention(*inputs).concat

    execute = torch.compile(run, fullgraph=True, dynamic=True)
    for lengths in ((3, 5), (5, 3), (3, 5)):
        case = nested_case(torch.float32, cuda, lengths=lengths, bias_kind="shared", prefix=(2,), transposed=True)
        q, k, v, mask, bias, leaves = build_nested(case, cuda)
        values = execute(q, k, v, mask, bias)
        upstream = torch.randn(values.shape, generator=torch.Generator().manual_seed(9))
        want_out, want = nested_oracle(case, upstream)
        assert_within(values, want_out, ATOL[torch.float32], f"out {lengths}")
        names = [n for n in ("q", "k", "v", "bias") if n in leaves]
        grads = torch.autograd.grad(values, [leaves[n] for n in names], upstream.to(cuda))
        for name, grad in zip(names, grads):
            assert_within(grad, want[name], ATOL[torch.float32] * max(1.0, float(want[name].abs().max())), f"d{name}")


def test_fake_tensor_mode_then_real(cuda):
    from torch._subclasses.fake_tensor import FakeTensorMode, is_fake

    with FakeTensorMode(allow_non_fake_inputs=True):
        q, k, v = (torch.randn(2, 4, 37, 2, 24, device=cuda, requires_grad=True) for _ in range(3))
        bias = torch.randn(2, 1, 2, 37, 37, device=cuda, requires_grad=True)
        mask = torch.rand(2, 4, 37, device=cuda) > 0.2
        out = triangle_attention(q, k, v, mask, bias)
        grads = torch.autograd.grad(out.sum(), (q, k, v, bias))
    assert is_fake(out) and out.shape == q.shape and out.dtype == q.dtype
    assert [g.shape for g in grads] == [q.shape, k.shape, v.shape, bias.shape] and all(is_fake(g) for g in grads)
    run_dense(dense_case(torch.float32, cols=37), cuda)


def test_golden_nested(cuda):
    g = torch.load(GOLDEN / "nested.pt", weights_only=False)
    for transposed, key in ((False, "packed"), (True, "packed_transposed")):
        els = g["elements"]
        pick = (lambda e, n: e[n].transpose(0, 1)) if transposed else (lambda e, n: e[n])
        q, k, v = (NestedTensor([pick(e, n).contiguous() for e in els], ragged_dims=(0, 1)) for n in "qkv")
        mask = NestedTensor([(e["mask"].t() if transposed else e["mask"]).contiguous() for e in els],
                            ragged_dims=(0, 1))
        bias = NestedTensor([(e["bias"].transpose(-2, -1) if transposed else e["bias"]).contiguous() for e in els],
                            ragged_dims=(2, 3))
        move = lambda n: n.packed_like(n.concat.to(cuda))  # noqa: E731
        q, k, v, mask, bias = (move(x) for x in (q, k, v, mask, bias))
        if transposed:
            q, k, v = (x.transpose(-4, -3) for x in (q, k, v))
            mask, bias = mask.transpose(-2, -1), bias.transpose(-2, -1)
        out = triangle_attention(q, k, v, mask, bias).concat
        assert_within(out, g[key], 1e-4, key)


# ------------------------------------------------------------------------------------------
# BASELINE configurations
# ------------------------------------------------------------------------------------------


def baseline_inputs(n, dtype, *, heads=4, dim=32, valid=None, seed=0, scale_inputs=0.5):
    gen = torch.Generator().manual_seed(seed)
    q, k, v = ((torch.randn(1, n, n, heads, dim, generator=gen) * scale_inputs).to(dtype) for _ in range(3))
    bias = torch.randn(1, 1, heads, n, n, generator=gen).to(dtype)
    upstream = torch.randn(1, n, n, heads, dim, generator=gen).to(dtype)
    if valid is None:
        mask = torch.ones(1, n, n, dtype=torch.bool)
    else:
        tok = torch.arange(n) < valid
        mask = (tok[:, None] & tok[None, :])[None]
    return q, k, v, bias, mask, upstream


def test_config2_forward_padding_mask(cuda):
    """BASELINE config 2: bf16 forward, N=384, 350 valid tokens; padded rows must be exactly zero."""
    q, k, v, bias, mask, _ = baseline_inputs(384, torch.bfloat16, valid=350)
    with torch.no_grad():
        out = triangle_attention(q.to(cuda), k.to(cuda), v.to(cuda), mask.to(cuda), bias.to(cuda))
    want = oracle.forward(q, k, v, mask, bias)
    assert_within(out, want, 2e-2, "out")
    assert torch.count_nonzero(out[:, 350:]) == 0


def test_config4_ending_node_ragged(cuda):
    """BASELINE config 4 at reduced lengths, where the oracle covers every row and every gradient (the full lengths
    with token masks are covered by test_config_parity_gpu.py):
    ending-node ragged batch, bf16, forward+backward, shared bias, all-valid masks."""
    case = nested_case(torch.bfloat16, cuda, lengths=(160, 100), heads=4, dim=32, bias_kind="shared",
                       transposed=True, seed=4)
    case["masks"] = [torch.ones_like(m) for m in case["masks"]]
    q, k, v, mask, bias, leaves = build_nested(case, cuda)
    values = triangle_attention(q, k, v, mask, bias).concat
    upstream = torch.randn(values.shape, generator=torch.Generator().manual_seed(5)).to(torch.bfloat16)
    want_out, want = nested_oracle(case, upstream)
    assert_within(values, want_out, 2e-2, "out")
    grads = torch.autograd.grad(values, [leaves[n] for n in ("q", "k", "v", "bias")], upstream.to(cuda))
    for name, grad in zip(("q", "k", "v", "bias"), grads):
        assert_within(grad, want[name], 2e-2 * max(1.0, float(want[name].abs().max())), f"d{name}")


@pytest.mark.parametrize(
    "n,valid,bias_kind",
    [(768, None, "shared"), (300, 260, "shared"), (200, 150, "none"), (136, None, "full"),
     (1000, 900, "shared"),   # 8 query tiles: two groups of 4, ragged last tile, f32 partial planes of dK and dV
     (1664, None, "none")],   # 13 query tiles: groups of 5, 5 and 3
)
def test_single_pass_reverse_matches_separate_kernels(cuda, n, valid, bias_kind):
    """Calls that want dQ, dK and dV take one kernel for all three (rows of more than 768 columns in groups of
    query tiles); the separate dQ and dK/dV kernels stay reachable through a flag.  Both must give the same
    gradients (same products, same rounding points; only the order of the f32 accumulation over tiles differs)."""
    q, k, v, bias, mask, upstream = baseline_inputs(n, torch.bfloat16, valid=valid, seed=21)
    if valid is not None:
        k[:, :, valid:] = float("inf")  # dropped keys may hold anything
        v[:, :, valid:] = float("nan")
    if bias_kind == "none":
        bias = None
    elif bias_kind == "full":
        bias = torch.randn(1, n, 4, n, n, generator=torch.Generator().manual_seed(5)).to(torch.bfloat16)
    dev = [None if t is None else t.to(cuda) for t in (q, k, v, bias)]
    results = []
    for split in (False, True):
        leaves = [t.detach().requires_grad_(True) for t in dev[:3]]
        with separate_reverse_kernels(split):
            out = triangle_attention(leaves[0], leaves[1], leaves[2], mask.to(cuda), dev[3])
            results.append(torch.autograd.grad(out, leaves, upstream.to(cuda)))
    live = slice(0, valid)
    for name, single, separate in zip(("dq", "dk", "dv"), *results):
        single, separate = single[:, live, live].float(), separate[:, live, live].float()
        assert torch.isfinite(single).all(), name
        assert_within(single, separate, 1e-2 * max(1.0, float(separate.abs().max())), name)


def test_config5_full_size_properties(cuda):
    """BASELINE config 5 at its full size (bf16 forward+backward, N=2048, all-ones mask).  The f32 oracle checks
    out/dq/dk/dv on a seeded sample of pair rows (rows are independent).  The shared-bias gradient, a sum over all
    2048 rows, is checked through size-independent properties: additivity over a split of the rows, bitwise
    repeatability, and agreement with the f32-accumulating layout-agnostic kernels on a quarter of the rows."""
    n = 2048
    q, k, v, bias, mask, upstream = baseline_inputs(n, torch.bfloat16, seed=11)
    dev = [t.to(cuda) for t in (q, k, v, bias)]
    mask_d, up_d = mask.to(cuda), upstream.to(cuda)
    leaves = [t.detach().requires_grad_(True) for t in dev]
    out = triangle_attention(leaves[0], leaves[1], leaves[2], mask_d, leaves[3])
    dq, dk, dv, db = torch.autograd.grad(out, leaves, up_d)
    rows = torch.randperm(n, generator=torch.Generator().manual_seed(2))[:3].sort().values
    want = oracle.forward_backward(q[:, rows], k[:, rows], v[:, rows], mask[:, rows], bias, upstream[:, rows])
    assert_within(out[:, rows], want[0], 2e-2, "out")
    for name, got, ref in (("dq", dq, want[1]), ("dk", dk, want[2]), ("dv", dv, want[3])):
        assert_within(got[:, rows], ref, 2e-2 * max(1.0, float(ref.abs().max())), name)
    assert torch.isfinite(db.float()).all()

    def bias_grad(rows_slice):
        b = dev[3].detach().requires_grad_(True)
        o = triangle_attention(dev[0][:, rows_slice], dev[1][:, rows_slice], dev[2][:, rows_slice], mask_d[:, rows_slice], b)
        return torch.autograd.grad(o, b, up_d[:, rows_slice])[0]

    tolerance = 2e-2 * max(1.0, float(db.float().abs().max()))
    halves = bias_grad(slice(0, n // 2)).float() + bias_grad(slice(n // 2, n)).float()
    assert_within(db.float(), halves, tolerance, "dbias additivity over rows")
    assert torch.equal(bias_grad(slice(0, n // 2)), bias_grad(slice(0, n // 2))), "dbias must be bitwise repeatable"
    quarter = slice(0, n // 4)
    with layout_agnostic_kernels():
        reference_quarter = bias_grad(quarter)
    assert_within(bias_grad(quarter), reference_quarter, 2e-2 * max(1.0, float(reference_quarter.float().abs().max())),
                  "dbias vs f32-accumulating kernels")


def test_padded_dense_equals_ragged(cuda):
    """The padded dense form (token masks) and the packed ragged form agree on the valid region."""
    lengths, heads, dim, n = (48, 29), 2, 32, 48
    case = nested_case(torch.bfloat16, cuda, lengths=lengths, heads=heads, dim=dim, bias_kind="shared", seed=6)
    case["masks"] = [torch.ones_like(m) for m in case["masks"]]
    q, k, v, mask, bias, _ = build_nested(case, cuda, requires_grad=False)
    ragged = torch.unbind(triangle_attention(q, k, v, mask, bias))
    dense = {name: torch.zeros(2, n, n, heads, dim, dtype=torch.bfloat16) for name in "qkv"}
    dense_bias = torch.zeros(2, 1, heads, n, n, dtype=torch.bfloat16)
    dense_mask = torch.zeros(2, n, n, dtype=torch.bool)
    for i, L in enumerate(lengths):
        for name in "qkv":
            dense[name][i, :L, :L] = case["elements"][name][i]
        dense_bias[i, :, :, :L, :L] = case["biases"][i]
        dense_mask[i, :L, :L] = True
    out = triangle_attention(dense["q"].to(cuda), dense["k"].to(cuda), dense["v"].to(cuda), dense_mask.to(cuda),
                             dense_bias.to(cuda))
    for i, L in enumerate(lengths):
        assert_within(out[i, :L, :L], ragged[i], 1e-2, f"sample {i}")
        assert torch.count_nonzero(out[i, L:]) == 0


# ------------------------------------------------------------------------------------------
# direct C-ABI call
# ------------------------------------------------------------------------------------------


@pytest.mark.parametrize("dtype,dim,cols", [(torch.float32, 24, 33), (torch.bfloat16, 32, 136)])
def test_c_abi_direct(cuda, dtype, dim, cols):
    """Forward and reverse passes through the raw C entry points, no autograd in between: once on the
    layout-agnostic f32 kernels, once on the tcgen05 kernels (16-bit, head size 32)."""
    from oops_b200.runtime import cabi

    lib = cabi.library()
    case = dense_case(dtype, dim=dim, cols=cols, bias_kind="shared", scale_inputs=1.0 if dtype is torch.float32 else 0.5)
    q, k, v, bias, up = (case[n].to(cuda) for n in ("q", "k", "v", "bias", "upstream"))
    mask = case["mask"].to(cuda)
    problem = cabi.make_problem(q, k, v, mask, bias, dim**-0.5)
    assert lib.oops_ta_supported(cabi.byref(problem)) == 0
    assert lib.oops_ta_uses_tensor_path(cabi.byref(problem), 1) == (1 if dtype is torch.bfloat16 else 0)
    atol = ATOL[dtype]
    scratch = torch.empty(int(lib.oops_ta_forward_workspace_bytes(cabi.byref(problem))) + 1, dtype=torch.uint8, device=cuda)
    problem.workspace, problem.workspace_bytes = scratch.data_ptr(), scratch.numel()
    out = torch.empty_like(q)
    lse = torch.empty(q.shape[0] * q.shape[1] * q.shape[3] * q.shape[2], dtype=torch.float32, device=cuda)
    stream = torch.cuda.current_stream().cuda_stream
    before = cabi.launch_count()
    out_pair = cabi.pair_of(out)
    assert lib.oops_ta_forward(cabi.byref(problem), cabi.byref(out_pair), lse.data_ptr(), stream) == 0
    assert cabi.launch_count() > before
    want = oracle_dense(case)
    assert_within(out, want[0], atol, "out")
    grads = cabi.Grads()
    dq, dk, dv, db = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v), torch.empty_like(bias)
    grads.dq, grads.dk, grads.dv = cabi.pair_of(dq), cabi.pair_of(dk), cabi.pair_of(dv)
    grads.dbias = db.data_ptr()
    grads.dbias_sb, grads.dbias_sg, grads.dbias_sh, grads.dbias_sq, grads.dbias_sk = db.stride()
    need = int(lib.oops_ta_backward_workspace_bytes(cabi.byref(problem), cabi.byref(grads)))
    scratch = torch.empty(need + 1, dtype=torch.uint8, device=cuda)
    problem.workspace, problem.workspace_bytes = scratch.data_ptr(), scratch.numel()
    dout_pair = cabi.pair_of(up)
    assert lib.oops_ta_backward(cabi.byref(problem), cabi.byref(out_pair), cabi.byref(dout_pair), lse.data_ptr(),
                                cabi.byref(grads), stream) == 0
    for name, got, ref in (("dq", dq, want[1]), ("dk", dk, want[2]), ("dv", dv, want[3]), ("dbias", db, want[4])):
        assert_within(got, ref, atol if dtype is torch.float32 else atol * max(1.0, float(ref.abs().max())), name)
    # a workspace that is too small is refused, not overrun
    if need > 16:
        problem.workspace_bytes = 16
        assert lib.oops_ta_backward(cabi.byref(problem), cabi.byref(out_pair), cabi.byref(dout_pair), lse.data_ptr(),
                                    cabi.byref(grads), stream) == 6
    torch.cuda.synchronize()


# ------------------------------------------------------------------------------------------
# device-side status word
# ------------------------------------------------------------------------------------------


def test_bounded_wait_that_runs_out_is_reported_and_cleared(cuda):
    """A device-side wait that gives up is reported by the status word, stops later tensor kernels until the word is
    cleared, and leaves the context usable.  The wait that runs out is the library's self-test kernel: one CTA waits
    one millisecond on a barrier that nothing completes, then tears down like a compute kernel and returns."""
    from oops_b200.attention.triangle.triangle_attention import checked_device_status
    from oops_b200.runtime import cabi

    lib = cabi.library()
    assert cabi.device_status(reset=True) == 0
    assert lib.oops_ta_selftest_wait_limit(torch.cuda.current_stream().cuda_stream) == 0
    assert cabi.device_status(reset=False) == cabi.STATUS_DEVICE_TIMEOUT
    case = dense_case(torch.bfloat16, dim=32, cols=72, bias_kind="shared", scale_inputs=0.5)
    args, _ = to_device(case, cuda, active=())
    # the word is still set: the forward tensor kernel returns at once, and a checked call says so (and clears it)
    with checked_device_status(), torch.no_grad(), pytest.raises(RuntimeError, match="device status 8"):
        triangle_attention(args["q"], args["k"], args["v"], args["mask"], args["bias"])
    assert cabi.device_status(reset=False) == 0
    # the next call is correct again
    with checked_device_status(), torch.no_grad():
        out = triangle_attention(args["q"], args["k"], args["v"], args["mask"], args["bias"])
    assert_within(out, oracle_dense(case)[0], 2e-2, "out after the status word was cleared")
