"""layer_norm on the GPU against the CPU oracle (float32 arithmetic cast to the activation dtype, the reference's own
check).  Cases and tolerances follow the reference's tests/normalization/layer_norm/test_layer_norm.py (:36-37
tolerances, :57-118 cases): dtypes, affine subsets, float32 ("master") parameters, strided / sliced / expanded
layouts, singleton and wide rows, packed ragged batches, which gradients are asked for."""

import pytest
import torch

import oops_b200 as oops
from oops_b200.runtime import cabi
from oracle import layer_norm_oracle as oracle

pytestmark = pytest.mark.gpu

TOL = {torch.float32: 1e-4, torch.float16: 3e-3, torch.bfloat16: 2e-2}          # forward, max-abs (reference :36)
GRAD_TOL = {torch.float32: 1e-4, torch.float16: 2e-2, torch.bfloat16: 4e-2}     # gradients (reference :37)


def _case(dtype, rows, width, affine, master, seed=40):
    gen = torch.Generator().manual_seed(seed)
    p_dtype = torch.float32 if master else dtype
    x = torch.randn(rows, width, generator=gen).to(dtype)
    w = (1 + 0.5 * torch.randn(width, generator=gen)).to(p_dtype) if affine in ("both", "weight") else None
    b = torch.randn(width, generator=gen).to(p_dtype) if affine in ("both", "bias") else None
    up = torch.randn(rows, width, generator=gen).to(dtype)
    return x, w, b, up


def _check(x, w, b, up, demand=(True, True, True), view=None):
    """Run the operator on (a view of) the inputs and compare everything that was asked for with the oracle."""
    dev = torch.device("cuda", 0)
    dtype = x.dtype
    xd = x.to(dev)
    if view == "transposed":   # rows strided, features contiguous is required: transposed leading axes of a 3-D view
        xd = xd.reshape(-1, 1, x.shape[-1]).expand(-1, 2, -1).transpose(0, 1)[0]
    elif view == "sliced":
        xd = torch.cat([xd, xd], dim=-1)[:, : x.shape[-1]]
    elif view == "expanded":
        xd = xd[:1].expand(x.shape[0], -1)
        x = x[:1].expand(x.shape[0], -1)
    xd = xd.detach().requires_grad_(demand[0])
    wd = w.to(dev).requires_grad_(demand[1]) if w is not None else None
    bd = b.to(dev).requires_grad_(demand[2]) if b is not None else None
    before = cabi.launch_count()
    out = oops.layer_norm(xd, x.shape[-1], wd, bd)
    assert cabi.launch_count() > before, "no kernel of the library was launched"
    assert out.dtype is dtype and out.shape == x.shape
    y, dx, dw, db = oracle.forward_backward(x.float(), None if w is None else w.float(), None if b is None else b.float(), up.float())
    assert float((out.detach().float().cpu() - y.to(dtype).float()).abs().max()) <= TOL[dtype]
    wanted = [(t, r) for t, r, d in ((xd, dx, demand[0]), (wd, dw, demand[1]), (bd, db, demand[2])) if t is not None and d]
    if not wanted:
        return
    grads = torch.autograd.grad(out, [t for t, _ in wanted], up.to(dev))
    for got, (leaf, ref) in zip(grads, wanted):
        assert got.dtype is leaf.dtype and got.shape == leaf.shape
        scale = max(1.0, float(ref.abs().max()))
        err = float((got.float().cpu() - ref.reshape(got.shape)).abs().max())
        assert err <= GRAD_TOL[dtype] * scale, f"gradient error {err:.3e} (largest value {scale:.3e})"


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("affine", ["both", "weight", "bias", "none"])
def test_dense(dtype, affine):
    _check(*_case(dtype, 67, 128, affine, master=False))


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_float32_parameters_with_16_bit_activations(dtype):
    _check(*_case(dtype, 67, 128, "both", master=True))


@pytest.mark.parametrize("rows,width", [(1, 8), (3, 32), (5, 33), (9, 1), (300, 1024), (7, 1025), (33, 4097), (17, 8192)])
def test_widths(rows, width):
    _check(*_case(torch.float32, rows, width, "both", master=False))
    _check(*_case(torch.bfloat16, rows, width, "both", master=True))


@pytest.mark.parametrize("view", ["transposed", "sliced", "expanded"])
def test_layouts(view):
    _check(*_case(torch.bfloat16, 12, 64, "both", master=True), view=view)


@pytest.mark.parametrize("demand", [(True, False, False), (False, True, False), (False, False, True)])
def test_single_gradient(demand):
    _check(*_case(torch.bfloat16, 40, 96, "both", master=False), demand=demand)


def test_parameter_gradients_are_reproducible_and_many_rows():
    """The pair tensor of config 3 (768 x 768 rows of 128 channels): every CTA contributes a partial row."""
    dev = torch.device("cuda", 0)
    x, w, b, up = (t.to(dev) if t is not None else None for t in _case(torch.bfloat16, 768 * 64, 128, "both", master=True))
    runs = []
    for _ in range(2):
        leaves = [t.detach().requires_grad_(True) for t in (x, w, b)]
        out = oops.layer_norm(leaves[0], 128, leaves[1], leaves[2])
        runs.append(torch.autograd.grad(out, leaves, up))
    for a, c in zip(*runs):
        assert torch.equal(a, c)
    _, _, dw, db = oracle.forward_backward(x.float().cpu(), w.cpu(), b.cpu(), up.float().cpu())
    assert float((runs[0][1].cpu() - dw).abs().max()) <= 4e-2 * max(1.0, float(dw.abs().max()))
    assert float((runs[0][2].cpu() - db).abs().max()) <= 4e-2 * max(1.0, float(db.abs().max()))


def test_nested():
    dev = torch.device("cuda", 0)
    gen = torch.Generator().manual_seed(7)
    parts = [torch.randn(n, 5, 32, generator=gen).to(torch.bfloat16).to(dev) for n in (3, 0, 7)]
    nested = oops.NestedTensor(parts, ragged_dims=(0,))
    w = torch.randn(32, generator=gen).to(dev)
    out = oops.layer_norm(nested, 32, w, None)
    for got, part in zip(torch.unbind(out), parts):
        want = oracle.layer_norm(part.float().cpu(), w.cpu(), None).to(torch.bfloat16)
        assert got.shape == part.shape
        if part.numel():
            assert float((got.float().cpu() - want.float()).abs().max()) <= TOL[torch.bfloat16]


def test_contract_on_gpu():
    dev = torch.device("cuda", 0)
    x = torch.ones(2, 8, device=dev)
    with pytest.raises(ValueError):
        oops.layer_norm(x, 8, torch.ones(8))  # parameters on another device
    with pytest.raises(oops.OOpsUnsupportedError):
        oops.layer_norm(x, 4)  # normalized_shape differs from the final dimension
    with pytest.raises(oops.OOpsUnsupportedError):
        oops.layer_norm(x.half(), 8, torch.ones(8, device=dev), torch.ones(8, device=dev).half())  # mixed parameter dtypes
    with pytest.raises(oops.OOpsUnsupportedError):
        oops.layer_norm(torch.empty(0, 8, device=dev), 8)
    with pytest.raises(oops.OOpsUnsupportedError):
        oops.layer_norm(torch.ones(2, 8193, device=dev), 8193)
