"""One process, two GPUs: calls on the second device after calls on the first (the reference's `secondary_cuda` cases,
tests/attention/triangle/test_triangle_attention.py:295-304).  Per-device state of the library (dynamic shared-memory
reservations, the status word, the static scratch array) must not leak from one device to the other."""

import pytest
import torch

import oops_b200 as oops
from oops_b200.runtime import cabi
from oracle import triangle_oracle as oracle

pytestmark = pytest.mark.gpu


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs in one process")
def test_forward_backward_on_both_devices_in_turn():
    gen = torch.Generator().manual_seed(3)
    n, h, d = 136, 4, 32
    q, k, v = ((torch.randn(1, n, n, h, d, generator=gen) * 0.5).bfloat16() for _ in range(3))
    bias = torch.randn(1, 1, h, n, n, generator=gen).bfloat16()
    up = torch.randn(1, n, n, h, d, generator=gen).bfloat16()
    want = oracle.forward_backward(q, k, v, None, bias, up)
    for index in (0, 1, 0, 1):
        dev = torch.device("cuda", index)
        leaves = [t.to(dev).requires_grad_(True) for t in (q, k, v, bias)]
        out = oops.triangle_attention(leaves[0], leaves[1], leaves[2], None, leaves[3])
        grads = torch.autograd.grad(out, leaves, up.to(dev))
        assert out.device == dev and all(g.device == dev for g in grads)
        for got, ref in zip((out, *grads), want):
            assert float((got.detach().float().cpu() - ref).abs().max()) <= 2e-2 * max(1.0, float(ref.abs().max()))
        x = torch.randn(40, 128, generator=gen).bfloat16()
        y = oops.layer_norm(x.to(dev), 128)
        assert y.device == dev and float((y.float().cpu() - torch.nn.functional.layer_norm(x.float(), (128,))).abs().max()) <= 2e-2
        with torch.cuda.device(dev):
            assert cabi.device_status(reset=False) == 0
