"""Row sharding with two CPU ranks over gloo: the sharded result equals the unsharded oracle.

The local attention is replaced by the PyTorch restatement (no GPU here), so this covers the
host logic of the multi-GPU path: shard bounds, the bias all-gather along the query axis and the
reduce-scatter of its gradient.
"""

from __future__ import annotations

import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oops_b200.distributed.row_shard import row_sharded_triangle_attention, shard_bounds
from oracle import triangle_oracle as oracle


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _inputs():
    gen = torch.Generator().manual_seed(0)
    n, h, d = 12, 2, 8
    q, k, v = (torch.randn(1, n, n, h, d, generator=gen) for _ in range(3))
    bias = torch.randn(1, 1, h, n, n, generator=gen)
    mask = torch.rand(1, n, n, generator=gen) > 0.2
    mask[..., 0] = True
    upstream = torch.randn(1, n, n, h, d, generator=gen)
    return q, k, v, bias, mask, upstream


def _worker(rank: int, world: int, port: int, results):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        q, k, v, bias, mask, upstream = _inputs()
        lo, hi = shard_bounds(q.shape[1], world, rank)
        leaves = [t[:, lo:hi].clone().requires_grad_(True) for t in (q, k, v)]
        bias_shard = bias[:, :, :, lo:hi].clone().requires_grad_(True)

        def local(query, key, value, m, b, scale=None):
            return oracle.reference_dense(query, key, value, m, b, scale)

        out = row_sharded_triangle_attention(*leaves, mask[:, lo:hi], bias_shard, attention=local)
        grads = torch.autograd.grad(out, [*leaves, bias_shard], upstream[:, lo:hi])
        results[rank] = [out.detach()] + [g.detach() for g in grads]
    finally:
        dist.destroy_process_group()


def test_two_ranks_match_unsharded():
    world = 2
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_worker, args=(world, _free_port(), results), nprocs=world, join=True)
    q, k, v, bias, mask, upstream = _inputs()
    want = oracle.forward_backward(q, k, v, mask, bias, upstream)
    for rank in range(world):
        lo, hi = shard_bounds(q.shape[1], world, rank)
        out, dq, dk, dv, db = results[rank]
        torch.testing.assert_close(out, want[0][:, lo:hi], atol=1e-5, rtol=1e-5)
        torch.testing.assert_close(dq, want[1][:, lo:hi], atol=1e-5, rtol=1e-5)
        torch.testing.assert_close(dk, want[2][:, lo:hi], atol=1e-5, rtol=1e-5)
        torch.testing.assert_close(dv, want[3][:, lo:hi], atol=1e-5, rtol=1e-5)
        torch.testing.assert_close(db, want[4][:, :, :, lo:hi], atol=1e-5, rtol=1e-5)


def test_shard_bounds():
    assert shard_bounds(2048, 8, 3) == (768, 1024)
    try:
        shard_bounds(10, 4, 0)
    except ValueError:
        pass
    else:
        raise AssertionError("uneven shards must be rejected")


def _ending_worker(rank: int, world: int, port: int, results):
    from oops_b200.distributed.row_shard import row_sharded_ending_node_attention

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        q, k, v, bias, mask, upstream = _inputs()
        lo, hi = shard_bounds(q.shape[1], world, rank)
        leaves = [t[:, lo:hi].clone().requires_grad_(True) for t in (q, k, v)]
        bias_shard = bias[:, :, :, lo:hi].clone().requires_grad_(True)

        def local(query, key, value, m, b, scale=None):
            return oracle.reference_dense(query, key, value, m, b, scale)

        out = row_sharded_ending_node_attention(*leaves, mask[:, lo:hi], bias_shard, attention=local)
        grads = torch.autograd.grad(out, [*leaves, bias_shard], upstream[:, lo:hi])
        results[rank] = [out.detach()] + [g.detach() for g in grads]
    finally:
        dist.destroy_process_group()


def test_ending_node_reshard_matches_unsharded():
    """Ending-node attention on a row-sharded pair tensor: re-shard to columns, attend on the transposed views,
    re-shard back; equals the unsharded ending-node call (the operator on the pair-axes transpose)."""
    world = 2
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_ending_worker, args=(world, _free_port(), results), nprocs=world, join=True)
    q, k, v, bias, mask, upstream = _inputs()
    leaves = [t.clone().requires_grad_(True) for t in (q, k, v, bias)]
    out = oracle.reference_dense(leaves[0].transpose(1, 2), leaves[1].transpose(1, 2), leaves[2].transpose(1, 2),
                                 mask.transpose(1, 2), leaves[3]).transpose(1, 2)
    want = [out.detach(), *torch.autograd.grad(out, leaves, upstream)]
    for rank in range(world):
        lo, hi = shard_bounds(q.shape[1], world, rank)
        got = results[rank]
        for name, g, w in zip(("out", "dq", "dk", "dv"), got[:4], want[:4]):
            torch.testing.assert_close(g, w[:, lo:hi], atol=1e-5, rtol=1e-5, msg=lambda m, name=name: f"{name}: {m}")
        torch.testing.assert_close(got[4], want[4][:, :, :, lo:hi], atol=1e-5, rtol=1e-5)
