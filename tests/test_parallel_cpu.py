"""Host-side logic of the two partitionings over gloo on CPU (world_size 2 and 3): shard ranges, the all-gather
re-assembly and the expert-parallel dispatch / combine against a single-process evaluation."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from eider_b200 import parallel


def test_shard_ranges_cover_and_align():
    for n, world in [(27648, 8), (5120, 8), (27648, 1), (13824, 4), (1280, 3)]:
        prev = 0
        for r in range(world):
            b, e = parallel.shard_range(n, world, r)
            assert b == prev and b % 128 == 0 and e % 128 == 0
            prev = e
        assert prev == n
    with pytest.raises(ValueError):
        parallel.shard_range(1000, 2, 0)


def test_gathered_to_row_major():
    g = torch.arange(2 * 3 * 4).reshape(2, 3, 4)
    y = parallel.gathered_to_row_major(g)
    assert y.shape == (3, 8)
    assert torch.equal(y[:, :4], g[0]) and torch.equal(y[:, 4:], g[1])


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _expert_fn_factory(rank, experts_per_rank):
    def fn(rows, local_expert):
        # expert e multiplies by (global id + 1) and adds its id: easy to evaluate without the exchange
        gid = local_expert.to(torch.float32) + rank * experts_per_rank
        return rows * (gid[:, None] + 1.0) + gid[:, None]
    return fn


def _worker(rank, world, port, tokens_per_rank, experts, k, hidden, result):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(1234 + rank)
        x = torch.randn(tokens_per_rank, hidden, generator=g)
        idx = torch.stack([torch.randperm(experts, generator=g)[:k] for _ in range(tokens_per_rank)])
        w = torch.rand(tokens_per_rank, k, generator=g)
        out = parallel.expert_parallel_moe(x, idx, w, experts, _expert_fn_factory(rank, experts // world))
        ref = torch.zeros_like(out)
        for slot in range(k):
            gid = idx[:, slot].to(torch.float32)
            ref += (x * (gid[:, None] + 1.0) + gid[:, None]) * w[:, slot:slot + 1]
        ok_moe = torch.allclose(out, ref, rtol=1e-5, atol=1e-5)

        # column-sharded linear with an f32 stand-in for the local slab
        n, kk = 128 * world * 2, 64
        wfull = torch.randn(n, kk, generator=torch.Generator().manual_seed(7))
        xin = torch.randn(5, kk, generator=torch.Generator().manual_seed(8))
        b, e = parallel.shard_range(n, world, rank)
        lin = parallel.ColumnShardedLinear(n, lambda t: t @ wfull[b:e].T)
        y = lin.forward(xin)
        ok_lin = torch.allclose(y, xin @ wfull.T, rtol=1e-5, atol=1e-5)
        result[rank] = int(ok_moe) + 2 * int(ok_lin)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_expert_parallel_and_column_shard_over_gloo(world):
    port = _free_port()
    ctx = mp.get_context("spawn")
    result = ctx.Manager().dict()
    procs = [ctx.Process(target=_worker, args=(r, world, port, 11 + r, 6 * world, 3, 16, result)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    assert dict(result) == {r: 3 for r in range(world)}


def test_single_process_matches_plain_evaluation():
    g = torch.Generator().manual_seed(0)
    x = torch.randn(9, 8, generator=g)
    idx = torch.stack([torch.randperm(4, generator=g)[:2] for _ in range(9)])
    w = torch.rand(9, 2, generator=g)
    out = parallel.expert_parallel_moe(x, idx, w, 4, _expert_fn_factory(0, 4))
    ref = sum((x * (idx[:, s:s + 1].float() + 1.0) + idx[:, s:s + 1].float()) * w[:, s:s + 1] for s in range(2))
    assert torch.allclose(out, ref, rtol=1e-5, atol=1e-5)
