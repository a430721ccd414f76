"""pair_bias_attention on the GPU against the CPU oracle: ranks 3 / 4 / 5+, key masks, bias broadcast over groups and
heads, gradients of q, k, v and the bias; the head-major operands reach the tcgen05 kernels as views (no copies)."""

import pytest
import torch

import oops_b200 as oops
from oops_b200.runtime import cabi
from oracle import pair_bias_oracle as oracle

pytestmark = pytest.mark.gpu

TOL = {torch.float32: 1e-4, torch.bfloat16: 2e-2, torch.float16: 2e-2}


def _run(shape, dtype, bias_shape=None, mask_shape=None, seed=0):
    """shape = (*prefix, S, H, N, D) (or rank 3 / 4); compares out, dq, dk, dv, dbias with the oracle's autograd."""
    dev = torch.device("cuda", 0)
    gen = torch.Generator().manual_seed(seed)
    q, k, v = ((torch.randn(shape, generator=gen) * 0.5).to(dtype) for _ in range(3))
    up = torch.randn(shape, generator=gen).to(dtype)
    bias = torch.randn(bias_shape, generator=gen).to(dtype) if bias_shape else None
    mask = None
    if mask_shape:
        mask = torch.rand(mask_shape, generator=gen) > 0.25
        mask[..., 0] = True
    leaves = [t.to(dev).requires_grad_(True) for t in (q, k, v)] + ([bias.to(dev).requires_grad_(True)] if bias is not None else [])
    before = cabi.launch_count()
    out = oops.pair_bias_attention(leaves[0], leaves[1], leaves[2], None if mask is None else mask.to(dev),
                                   leaves[3] if bias is not None else None)
    assert cabi.launch_count() > before
    assert out.shape == q.shape and out.dtype is dtype
    grads = torch.autograd.grad(out, leaves, up.to(dev))

    ref_leaves = [t.double().requires_grad_(True) for t in (q, k, v)] + ([bias.double().requires_grad_(True)] if bias is not None else [])
    rank = len(shape)
    key_mask = None
    if mask is not None:
        key_mask = mask[..., None, None, :] if rank >= 4 else mask[None, None, :]
    ref_bias = ref_leaves[3] if bias is not None else None
    want = oracle.pair_bias_attention(ref_leaves[0], ref_leaves[1], ref_leaves[2], key_mask, ref_bias, dtype=torch.float64)
    want_grads = torch.autograd.grad(want, ref_leaves, up.double())
    tol = TOL[dtype]
    assert float((out.detach().double().cpu() - want.detach()).abs().max()) <= tol
    for got, ref in zip(grads, want_grads):
        assert got.shape == ref.shape
        assert float((got.double().cpu() - ref).abs().max()) <= tol * max(1.0, float(ref.abs().max()))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_rank5_tensor_path_shapes(dtype):
    # D = 32 with 16-bit operands takes the tcgen05 kernels on the permuted views
    _run((2, 3, 4, 160, 32), dtype, bias_shape=(2, 1, 4, 160, 160), mask_shape=(2, 3, 160))


def test_rank4_bias_per_group_and_shared_mask():
    _run((3, 2, 40, 32), torch.bfloat16, bias_shape=(3, 2, 40, 40), mask_shape=(1, 40), seed=1)


def test_rank3_broadcast_heads():
    _run((4, 33, 16), torch.float32, bias_shape=(1, 33, 33), mask_shape=(33,), seed=2)


def test_prefix_axes_and_no_bias():
    _run((2, 2, 1, 2, 24, 8), torch.float32, mask_shape=(2, 2, 1, 24), seed=3)


def test_views_reach_the_tensor_kernels_without_copies():
    dev = torch.device("cuda", 0)
    q = torch.randn(1, 2, 4, 128, 32, device=dev, dtype=torch.bfloat16)
    bias = torch.randn(1, 1, 4, 128, 128, device=dev, dtype=torch.bfloat16)
    pairs = q.permute(0, 1, 3, 2, 4)  # what the wrapper hands to triangle_attention
    assert pairs.data_ptr() == q.data_ptr() and pairs.stride(-1) == 1
    problem = cabi.make_problem(pairs, pairs, pairs, None, bias, 32**-0.5)
    assert cabi.library().oops_ta_uses_tensor_path(cabi.byref(problem), 1) == 1, "head-major views must take the tcgen05 kernels"
    out = oops.pair_bias_attention(q, q, q, pair_bias=bias)
    assert out.is_contiguous() and out.shape == q.shape
