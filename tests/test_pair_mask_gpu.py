"""pair_mask_from_token_mask on packed ragged batches (CUDA kernel behind oops_ta_pair_mask_packed) against the
reference's own formula per sample (tests/mask/test_pair_mask_from_token_mask.py:30-33, :54-71 in the reference)."""

import pytest
import torch

import oops_b200 as oops
from oops_b200.runtime import cabi

pytestmark = pytest.mark.gpu


def _reference(mask):
    token = mask.bool()
    return token[..., :, None] & token[..., None, :]


def _check(parts):
    before = cabi.launch_count()
    actual = oops.pair_mask_from_token_mask(oops.NestedTensor(parts, ragged_dims=(0,)))
    expected = torch.cat([_reference(p).flatten() for p in parts])
    assert actual.concat.dtype is torch.bool
    torch.testing.assert_close(actual.concat, expected, atol=0, rtol=0)
    for got, part in zip(torch.unbind(actual), parts):
        torch.testing.assert_close(got, _reference(part), atol=0, rtol=0)
    return cabi.launch_count() - before


@pytest.mark.parametrize("dtype", [torch.bool, torch.float32, torch.int64])
def test_small(dtype):
    device = torch.device("cuda", 0)
    parts = [torch.tensor([1, 0]).to(device=device, dtype=dtype), torch.tensor([-2, 0, 3]).to(device=device, dtype=dtype)]
    assert _check(parts) == 1


def test_empty_elements():
    device = torch.device("cuda", 0)
    parts = [torch.empty(0, dtype=torch.bool, device=device), torch.empty(0, dtype=torch.bool, device=device)]
    assert _check(parts) == 0
    assert _check([parts[0], torch.tensor([True, False, True], device=device)]) == 1


def test_ragged_lengths_of_config_4():
    """Lengths (1024, 700) plus odd ones: rows that end inside a 16-cell chunk, unaligned sample starts."""
    device = torch.device("cuda", 0)
    gen = torch.Generator().manual_seed(3)
    parts = [(torch.rand(n, generator=gen) > 0.3).to(device) for n in (1024, 700, 1, 17, 33, 255)]
    assert _check(parts) == 1


def test_result_is_a_mask_for_triangle_attention():
    device = torch.device("cuda", 0)
    tok = (torch.arange(40) < 33).to(device)
    pair = oops.pair_mask_from_token_mask(tok[None])
    q = torch.randn(1, 40, 40, 2, 32, device=device, dtype=torch.bfloat16)
    out = oops.triangle_attention(q, q, q, pair)
    assert torch.isfinite(out.float()).all()
