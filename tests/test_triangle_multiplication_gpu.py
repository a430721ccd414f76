"""triangle_multiplication (this library's layer norm + library GEMMs) against the CPU oracle, both directions, with and
without mask and projection biases, forward and gradients.  Tolerances of the reference's own test
(tests/pair/triangle_multiplication/test_triangle_multiplication.py): f32 1e-4 class, bf16 a few 1e-2."""

import pytest
import torch

import oops_b200 as oops
from oracle import triangle_multiplication_oracle as oracle

pytestmark = pytest.mark.gpu


def _weights(gen, channels, hidden, biases):
    def t(*shape, scale=1.0):
        return torch.randn(*shape, generator=gen) * scale
    w = dict(input_norm_weight=1 + 0.1 * t(channels), input_norm_bias=0.1 * t(channels),
             left_value_weight=t(hidden, channels, scale=channels**-0.5), left_gate_weight=t(hidden, channels, scale=channels**-0.5),
             right_value_weight=t(hidden, channels, scale=channels**-0.5), right_gate_weight=t(hidden, channels, scale=channels**-0.5),
             output_norm_weight=1 + 0.1 * t(hidden), output_norm_bias=0.1 * t(hidden),
             output_weight=t(channels, hidden, scale=hidden**-0.5), output_gate_weight=t(channels, channels, scale=channels**-0.5))
    if biases:
        w.update(left_value_bias=0.1 * t(hidden), left_gate_bias=0.1 * t(hidden), right_value_bias=0.1 * t(hidden),
                 right_gate_bias=0.1 * t(hidden), output_bias=0.1 * t(channels), output_gate_bias=0.1 * t(channels))
    return w


@pytest.mark.parametrize("direction", ["outgoing", "incoming"])
@pytest.mark.parametrize("dtype,biases,masked", [(torch.float32, True, True), (torch.float32, False, False), (torch.bfloat16, True, True)])
def test_against_oracle(direction, dtype, biases, masked):
    dev = torch.device("cuda", 0)
    gen = torch.Generator().manual_seed(0)
    tokens, channels, hidden = 24, 32, 48
    pair = torch.randn(2, tokens, tokens, channels, generator=gen).to(dtype)
    mask = (torch.rand(2, tokens, tokens, generator=gen) > 0.2).float() if masked else None
    weights = _weights(gen, channels, hidden, biases)
    up = torch.randn(2, tokens, tokens, channels, generator=gen).to(dtype)

    pair_d = pair.to(dev).requires_grad_(True)
    weights_d = {k: v.to(dev).requires_grad_(True) for k, v in weights.items()}
    out = oops.triangle_multiplication(pair_d, None if mask is None else mask.to(dev), direction=direction, **weights_d)
    assert out.shape == pair.shape and out.dtype is dtype
    grads = torch.autograd.grad(out, [pair_d, *weights_d.values()], up.to(dev))

    pair_r = pair.double().requires_grad_(True)
    weights_r = {k: v.double().requires_grad_(True) for k, v in weights.items()}
    want = oracle.triangle_multiplication(pair_r, mask, direction=direction, dtype=torch.float64, **weights_r)
    want_grads = torch.autograd.grad(want, [pair_r, *weights_r.values()], up.double())
    tol = 2e-4 if dtype is torch.float32 else 6e-2
    assert float((out.detach().double().cpu() - want.detach()).abs().max()) <= tol * max(1.0, float(want.detach().abs().max()))
    for got, ref in zip(grads, want_grads):
        assert float((got.double().cpu() - ref).abs().max()) <= tol * max(1.0, float(ref.abs().max()))


def test_contract():
    dev = torch.device("cuda", 0)
    gen = torch.Generator().manual_seed(1)
    weights = {k: v.to(dev) for k, v in _weights(gen, 8, 12, False).items()}
    pair = torch.ones(4, 4, 8, device=dev)
    with pytest.raises(ValueError):
        oops.triangle_multiplication(pair, direction="sideways", **weights)
    with pytest.raises(ValueError):
        oops.triangle_multiplication(torch.ones(4, 5, 8, device=dev), **weights)
    with pytest.raises(ValueError):
        oops.triangle_multiplication(pair, **{**weights, "output_weight": torch.ones(8, 11, device=dev)})
