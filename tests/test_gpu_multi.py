"""Two-rank NCCL checks of the partitioned configs (skipped with fewer than two GPUs): the N-sharded GEMM + all-gather
equals the unsharded GEMM bit for bit, and the expert-parallel MoE equals the single-GPU pipeline."""
import os
import socket

import pytest

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, result):
    import torch
    import torch.distributed as dist

    from eider_b200 import ops, parallel
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        # ---- dense: N-sharded NVFP4 GEMM + all-gather vs the whole GEMM on every rank
        m, n, k = 256, 1024, 1024
        g = torch.Generator(device="cuda").manual_seed(5)
        w = torch.randn(n, k, device="cuda", generator=g) * 0.02
        x = torch.randn(m, k, device="cuda", generator=g).to(torch.bfloat16)
        full = ops.ModelOptWeight.quantize(w)
        xq = ops.quantize_nvfp4_rowscale(x)
        y_ref = ops.Fp4TnMatmulPlan(m, n, k).run(xq, full)
        b, e = parallel.shard_range(n, world, rank)
        shard = ops.ModelOptWeight.from_checkpoint(full.packed[b:e].contiguous(), full.scales_row_major[b:e].contiguous(),
                                                   full.weight_scale_2)
        plan = ops.Fp4TnMatmulPlan(m, e - b, k)
        lin = parallel.ColumnShardedLinear(n, lambda t: plan.run(ops.quantize_nvfp4_rowscale(t), shard))
        y = lin.forward(x)
        ok_dense = bool(torch.equal(y, y_ref))
        # the same through the fused all-gather: the GEMM epilogue writes this rank's columns into every rank's output
        plan_fused = ops.Fp4TnMatmulPlan(m, e - b, k)
        lin_fused = parallel.ColumnShardedLinear(n, lambda t: plan_fused.run(ops.quantize_nvfp4_rowscale(t), shard))
        lin_fused.fuse_into(plan_fused, m)
        for code in (0, 512):  # plain peer stores (tile shape chosen by the plan), then CTA pairs with TMA stores to the peers
            if code:
                plan_fused.set_block_n(code)
            for _ in range(3):  # repeated steps reuse the symmetric buffer
                y_fused = lin_fused.forward(x)
            torch.cuda.synchronize()
            ok_dense = ok_dense and bool(torch.equal(y_fused, y_ref)) and plan_fused.status() == 0

        # ---- MoE: expert parallel vs single GPU
        tokens, experts, top_k, hidden, inter = 64 * world, 8, 2, 256, 128
        g = torch.Generator(device="cuda").manual_seed(9)
        xs = torch.randn(tokens, hidden, device="cuda", generator=g).to(torch.bfloat16)
        logits = torch.randn(tokens, experts, device="cuda", generator=g)
        wgu = torch.randn(experts, 2 * inter, hidden, device="cuda", generator=g) * 0.02
        wdn = torch.randn(experts, hidden, inter, device="cuda", generator=g) * 0.02
        w_gu, w_dn = ops.GroupedNvfp4Weights.quantize(wgu), ops.GroupedNvfp4Weights.quantize(wdn)
        ref = ops.GroupedMoe(tokens, experts, top_k, hidden, inter).run(xs, logits, w_gu, w_dn).clone()
        per = experts // world
        sl = slice(rank * per, (rank + 1) * per)
        local = parallel.LocalExperts(
            ops.GroupedNvfp4Weights.from_checkpoint(w_gu.packed[sl].contiguous(), w_gu.scales_row_major[sl].contiguous(), w_gu.alpha[sl]),
            ops.GroupedNvfp4Weights.from_checkpoint(w_dn.packed[sl].contiguous(), w_dn.scales_row_major[sl].contiguous(), w_dn.alpha[sl]),
            hidden, inter)
        tl = tokens // world
        rows = slice(rank * tl, (rank + 1) * tl)
        idx, wts = ops.moe_topk(logits[rows].contiguous(), top_k, True)
        out = parallel.expert_parallel_moe(xs[rows].contiguous(), idx, wts, experts, local,
                                           combine_fn=parallel.device_combine(tl, top_k))
        torch.cuda.synchronize()
        ok_moe = bool(torch.allclose(out, ref[rows], rtol=1e-5, atol=1e-6))
        result[rank] = (ok_dense, ok_moe)
    finally:
        dist.destroy_process_group()


def test_two_rank_partitioned_paths():
    torch = pytest.importorskip("torch")
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    result = ctx.Manager().dict()
    procs = [ctx.Process(target=_worker, args=(r, world, port, result)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=300)
        assert p.exitcode == 0
    assert dict(result) == {0: (True, True), 1: (True, True)}
