"""Row sharding on real GPUs over NCCL: every rank's shard of the output and of all four gradients equals the
single-GPU call on the same inputs.  Needs two or more GPUs on the node; skipped otherwise (the host logic is
covered on CPU by test_row_shard_gloo.py)."""

from __future__ import annotations

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oops_b200.distributed.row_shard import row_sharded_triangle_attention, shard_bounds

pytestmark = pytest.mark.gpu


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _inputs(n=256, h=4, d=32):
    gen = torch.Generator().manual_seed(3)
    q, k, v = ((torch.randn(1, n, n, h, d, generator=gen) * 0.5).to(torch.bfloat16) for _ in range(3))
    bias = torch.randn(1, 1, h, n, n, generator=gen).to(torch.bfloat16)
    mask = torch.rand(1, n, n, generator=gen) > 0.1
    mask[..., 0] = True
    upstream = torch.randn(1, n, n, h, d, generator=gen).to(torch.bfloat16)
    return q, k, v, bias, mask, upstream


def _worker(rank: int, world: int, port: int, results):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    device = torch.device("cuda", rank)
    torch.cuda.set_device(device)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    try:
        q, k, v, bias, mask, upstream = _inputs()
        lo, hi = shard_bounds(q.shape[1], world, rank)
        leaves = [t[:, lo:hi].to(device).requires_grad_(True) for t in (q, k, v)]
        bias_shard = bias[:, :, :, lo:hi].to(device).requires_grad_(True)
        out = row_sharded_triangle_attention(*leaves, mask[:, lo:hi].to(device), bias_shard)
        grads = torch.autograd.grad(out, [*leaves, bias_shard], upstream[:, lo:hi].to(device))
        torch.cuda.synchronize()
        results[rank] = [out.detach().cpu()] + [g.detach().cpu() for g in grads]
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_ranks_match_single_gpu(cuda):
    from oops_b200 import triangle_attention

    world = min(4, torch.cuda.device_count())
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_worker, args=(world, _free_port(), results), nprocs=world, join=True)
    q, k, v, bias, mask, upstream = _inputs()
    leaves = [t.to(cuda).requires_grad_(True) for t in (q, k, v, bias)]
    out = triangle_attention(leaves[0], leaves[1], leaves[2], mask.to(cuda), leaves[3])
    dq, dk, dv, db = (g.cpu() for g in torch.autograd.grad(out, leaves, upstream.to(cuda)))
    out = out.detach().cpu()
    for rank in range(world):
        lo, hi = shard_bounds(q.shape[1], world, rank)
        got = results[rank]
        # rows are independent: the per-row results are the same kernels on the same data
        assert torch.equal(got[0], out[:, lo:hi]), f"rank {rank} out"
        assert torch.equal(got[1], dq[:, lo:hi]) and torch.equal(got[2], dk[:, lo:hi]) and torch.equal(got[3], dv[:, lo:hi])
        # the bias gradient sums rows in a different grouping (per rank, then across ranks): bf16 rounding differs
        scale = max(1.0, float(db.float().abs().max()))
        assert float((got[4].float() - db[:, :, :, lo:hi].float()).abs().max()) <= 2e-2 * scale, f"rank {rank} dbias"


def _ending_worker(rank: int, world: int, port: int, results):
    from oops_b200.distributed.row_shard import row_sharded_ending_node_attention

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    device = torch.device("cuda", rank)
    torch.cuda.set_device(device)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    try:
        q, k, v, bias, mask, upstream = _inputs()
        lo, hi = shard_bounds(q.shape[1], world, rank)
        leaves = [t[:, lo:hi].to(device).requires_grad_(True) for t in (q, k, v)]
        bias_shard = bias[:, :, :, lo:hi].to(device).requires_grad_(True)
        out = row_sharded_ending_node_attention(*leaves, mask[:, lo:hi].to(device), bias_shard)
        grads = torch.autograd.grad(out, [*leaves, bias_shard], upstream[:, lo:hi].to(device))
        torch.cuda.synchronize()
        results[rank] = [out.detach().cpu()] + [g.detach().cpu() for g in grads]
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_ending_node_ranks_match_single_gpu(cuda):
    """Ending-node attention on a row-sharded pair tensor (all-to-all to column ownership, attention on the transposed
    views, all-to-all back) against the single-GPU ending-node call."""
    from oops_b200 import triangle_attention

    world = min(4, torch.cuda.device_count())
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_ending_worker, args=(world, _free_port(), results), nprocs=world, join=True)
    q, k, v, bias, mask, upstream = _inputs()
    leaves = [t.to(cuda).requires_grad_(True) for t in (q, k, v, bias)]
    out = triangle_attention(leaves[0].transpose(1, 2), leaves[1].transpose(1, 2), leaves[2].transpose(1, 2),
                             mask.to(cuda).transpose(1, 2), leaves[3]).transpose(1, 2)
    dq, dk, dv, db = (g.cpu() for g in torch.autograd.grad(out, leaves, upstream.to(cuda)))
    out = out.detach().cpu()
    for rank in range(world):
        lo, hi = shard_bounds(q.shape[1], world, rank)
        got = results[rank]
        assert torch.equal(got[0], out[:, lo:hi]), f"rank {rank} out"
        assert torch.equal(got[1], dq[:, lo:hi]) and torch.equal(got[2], dk[:, lo:hi]) and torch.equal(got[3], dv[:, lo:hi])
        scale = max(1.0, float(db.float().abs().max()))
        assert float((got[4].float() - db[:, :, :, lo:hi].float()).abs().max()) <= 2e-2 * scale, f"rank {rank} dbias"
