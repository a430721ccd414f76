"""The pair-bias oracle against F.scaled_dot_product_attention (the reference's composed form,
oops/attention/pair_bias/composed.py:32-58) and the wrapper's argument contract (no GPU)."""

import pytest
import torch
from torch.nn import functional as F

import oops_b200 as oops
from oracle import pair_bias_oracle as oracle


def test_oracle_matches_sdpa():
    gen = torch.Generator().manual_seed(3)
    q, k, v = (torch.randn(2, 3, 4, 9, 8, generator=gen, dtype=torch.float64) for _ in range(3))
    bias = torch.randn(2, 1, 4, 9, 9, generator=gen, dtype=torch.float64)
    keep = torch.rand(2, 3, 9, generator=gen) > 0.3
    keep[..., 0] = True
    want = F.scaled_dot_product_attention(q, k, v, attn_mask=bias.masked_fill(~keep[:, :, None, None, :], float("-inf")))
    got = oracle.pair_bias_attention(q, k, v, keep[:, :, None, None, :], bias, dtype=torch.float64)
    torch.testing.assert_close(got, want, atol=1e-12, rtol=1e-12)


def test_fully_masked_rows_are_zero():
    q = torch.randn(1, 2, 4, 8)
    keep = torch.zeros(1, 1, 1, 4, dtype=torch.bool)
    assert torch.equal(oracle.pair_bias_attention(q, q, q, keep, None), torch.zeros_like(q))


def test_contract():
    q = torch.ones(2, 4, 8)
    with pytest.raises(ValueError):
        oops.pair_bias_attention(torch.ones(4, 8), torch.ones(4, 8), torch.ones(4, 8))
    with pytest.raises(oops.OOpsUnsupportedError):
        oops.pair_bias_attention(q, torch.ones(2, 5, 8), torch.ones(2, 5, 8))  # different key length
    with pytest.raises(oops.OOpsUnsupportedError):
        oops.pair_bias_attention(q, q, q, mask=torch.ones(4, 4, dtype=torch.bool))  # a mask with a query axis
    with pytest.raises(ValueError):
        oops.pair_bias_attention(q, q, q, pair_bias=torch.ones(3, 4, 4))  # heads neither 1 nor H
    with pytest.raises(oops.OOpsUnsupportedError):
        oops.pair_bias_attention(q, q, q, pair_bias=torch.ones(2, 1, 4))  # singleton query axis
    with pytest.raises(oops.OOpsUnsupportedError):
        oops.pair_bias_attention(q, q, q)  # CPU operands: no fallback
