"""pair_mask_from_token_mask: dense results and argument contract (no GPU).

Cases follow the reference's tests/mask/test_pair_mask_from_token_mask.py (:30-33 reference formula, :47-52 dense
dtypes, :73-88 contract)."""

import pytest
import torch

import oops_b200 as oops


def _reference(mask):
    token = mask.bool()
    return token[..., :, None] & token[..., None, :]


@pytest.mark.parametrize("dtype", [torch.bool, torch.int64, torch.float32])
def test_dense(dtype):
    mask = torch.tensor([[1, 0, 2], [0, -1, 3]], dtype=dtype)
    actual = oops.pair_mask_from_token_mask(mask)
    assert actual.dtype is torch.bool
    torch.testing.assert_close(actual, _reference(mask), atol=0, rtol=0)


def test_dense_feeds_triangle_attention_shape():
    tok = torch.arange(12) < 9
    assert oops.pair_mask_from_token_mask(tok[None]).shape == (1, 12, 12)


@pytest.mark.parametrize("case", ["rank", "cpu_nested", "complex", "nested_rank"])
def test_contract(case):
    if case == "rank":
        with pytest.raises(ValueError):
            oops.pair_mask_from_token_mask(torch.tensor(True))
        return
    shape = (2, 1) if case == "nested_rank" else (2,)
    dtype = torch.complex64 if case == "complex" else torch.bool
    mask = oops.NestedTensor([torch.ones(shape, dtype=dtype)], ragged_dims=(0,))
    error = ValueError if case == "nested_rank" else oops.OOpsUnsupportedError
    with pytest.raises(error):
        oops.pair_mask_from_token_mask(mask)
