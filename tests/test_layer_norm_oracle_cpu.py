"""The layer-norm oracle against F.layer_norm in float32, which is the reference's own check
(tests/normalization/layer_norm/test_layer_norm.py:207-219 in the reference), and the operator's argument contract."""

import pytest
import torch
from torch.nn import functional as F

import oops_b200 as oops
from oracle import layer_norm_oracle as oracle


@pytest.mark.parametrize("affine", ["both", "weight", "bias", "none"])
@pytest.mark.parametrize("shape", [(3, 32), (67, 128), (2, 5, 8), (1, 1)])
def test_oracle_matches_functional(affine, shape):
    gen = torch.Generator().manual_seed(40)
    width = shape[-1]
    x = torch.randn(shape, generator=gen, dtype=torch.float64, requires_grad=True)
    w = torch.randn(width, generator=gen, dtype=torch.float64, requires_grad=True) if affine in ("both", "weight") else None
    b = torch.randn(width, generator=gen, dtype=torch.float64, requires_grad=True) if affine in ("both", "bias") else None
    up = torch.randn(shape, generator=gen, dtype=torch.float64)
    want = F.layer_norm(x, (width,), w, b)
    leaves = [t for t in (x, w, b) if t is not None]
    grads = list(torch.autograd.grad(want, leaves, up))
    y, dx, dw, db = oracle.forward_backward(x.detach(), None if w is None else w.detach(), None if b is None else b.detach(), up,
                                            dtype=torch.float64)
    torch.testing.assert_close(y, want.detach(), atol=1e-12, rtol=1e-12)
    torch.testing.assert_close(oracle.layer_norm(x.detach(), w, b, dtype=torch.float64), want.detach(), atol=1e-12, rtol=1e-12)
    torch.testing.assert_close(dx, grads.pop(0), atol=1e-10, rtol=1e-10)
    if w is not None:
        torch.testing.assert_close(dw, grads.pop(0), atol=1e-10, rtol=1e-10)
    if b is not None:
        torch.testing.assert_close(db, grads.pop(0), atol=1e-10, rtol=1e-10)


def test_contract_without_gpu():
    with pytest.raises(oops.OOpsUnsupportedError):
        oops.layer_norm(torch.ones(2, 8), 8)  # CPU activations
    with pytest.raises(oops.OOpsUnsupportedError):
        oops.layer_norm(torch.ones(2, 4, 8), (4, 8))  # more than the final dimension
    nested = oops.NestedTensor([torch.ones(3, 8), torch.ones(2, 8)], ragged_dims=(0,))
    with pytest.raises(ValueError):
        oops.layer_norm(nested, 8, weight=nested)
    with pytest.raises(oops.OOpsUnsupportedError):
        oops.layer_norm(nested.transpose(1, 2), 3)  # the feature axis must be static and physically last
