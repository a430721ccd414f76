"""Repeated calls give bit-identical outputs and gradients (the reference promises reproducible gradients: no
floating-point atomics).  A rare race in a kernel shows up here as one differing tensor."""

import pytest
import torch

from oops_b200 import triangle_attention
from oops_b200.runtime import cabi

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("rows,n,masked", [(96, 768, False), (40, 2048, False), (64, 1000, True)])
def test_repeated_calls_are_bit_identical(rows, n, masked):
    dev = torch.device("cuda", 0)
    gen = torch.Generator().manual_seed(1)
    q, k, v = ((torch.randn(1, rows, n, 4, 32, generator=gen) * 0.5).bfloat16().to(dev) for _ in range(3))
    up = torch.randn(1, rows, n, 4, 32, generator=gen).bfloat16().to(dev)
    bias = torch.randn(1, 1, 4, n, n, generator=gen).bfloat16().to(dev)
    mask = (torch.rand(1, rows, n, generator=gen) > 0.1).to(dev) if masked else None
    first = None
    for _ in range(12):
        leaves = [t.detach().requires_grad_(True) for t in (q, k, v, bias)]
        out = triangle_attention(leaves[0], leaves[1], leaves[2], mask, leaves[3])
        result = [out.detach(), *torch.autograd.grad(out, leaves, up)]
        if first is None:
            first = [r.clone() for r in result]
            continue
        for name, a, b in zip(("out", "dq", "dk", "dv", "dbias"), first, result):
            assert torch.equal(a, b), f"{name} changed between two calls on the same inputs"
    assert cabi.device_status(reset=False) == 0
