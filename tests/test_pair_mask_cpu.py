"""pair_mask_from_token_mask without a GPU: dense results for several dtypes and ranks, and the argument contract
(what the reference's tests/mask/test_pair_mask_from_token_mask.py checks on the dense arm and for refusals)."""

import pytest
import torch

import oops_b200 as oops


def _outer_and(tokens):
    valid = tokens != 0
    return valid.unsqueeze(-1) & valid.unsqueeze(-2)


@pytest.mark.parametrize("dtype", [torch.bool, torch.int64, torch.float32, torch.uint8])
@pytest.mark.parametrize("shape", [(5,), (2, 3), (2, 1, 7)])
def test_dense_matches_the_outer_conjunction(dtype, shape):
    gen = torch.Generator().manual_seed(11)
    tokens = (torch.randint(-2, 3, shape, generator=gen)).to(dtype) if dtype is not torch.bool else torch.rand(shape, generator=gen) > 0.4
    got = oops.pair_mask_from_token_mask(tokens)
    assert got.dtype is torch.bool and got.shape == (*shape, shape[-1])
    assert torch.equal(got, _outer_and(tokens))


def test_dense_result_is_a_triangle_attention_mask():
    tokens = torch.arange(12) < 9
    assert oops.pair_mask_from_token_mask(tokens[None]).shape == (1, 12, 12)


def test_scalar_is_refused():
    with pytest.raises(ValueError):
        oops.pair_mask_from_token_mask(torch.tensor(True))


@pytest.mark.parametrize("kind,error", [("cpu", oops.OOpsUnsupportedError), ("complex", oops.OOpsUnsupportedError), ("rank", ValueError)])
def test_packed_batches_are_refused_when_unservable(kind, error):
    element = torch.ones((2, 1) if kind == "rank" else (2,), dtype=torch.complex64 if kind == "complex" else torch.bool)
    with pytest.raises(error):
        oops.pair_mask_from_token_mask(oops.NestedTensor([element], ragged_dims=(0,)))
