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
        # plain peer stores (tile shape chosen by the plan), CTA pairs with one multicast store per tile (when the box
        # offers an NVLink multicast mapping), CTA pairs with one TMA store per peer
        # (384: the 256 x 192 form of the pair kernel, three 64-column steps per tile through the same staging buffers)
        for code, use_multicast in ((0, False), (512, True), (512, False), (384, True), (384, False)):
            if code:
                plan_fused.set_block_n(code)
            if not use_multicast:
                plan_fused.set_output_multicast(0)
            elif not lin_fused.multicast:
                continue
            for _ in range(3):  # repeated steps reuse the symmetric buffer
                y_fused = lin_fused.forward(x).clone()
            torch.cuda.synchronize()
            lin_fused.check()
            ok_dense = ok_dense and bool(torch.equal(y_fused, y_ref)) and plan_fused.status() == 0
            y_fused.zero_()

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
        # the same layer over peer memory: NVFP4 rows dispatched and bf16 rows returned by peer stores, counts on the device,
        # bounded device barriers between the phases; equals the single-GPU pipeline bit for bit, step after step
        local_gu = ops.GroupedNvfp4Weights.from_checkpoint(w_gu.packed[sl].contiguous(), w_gu.scales_row_major[sl].contiguous(), w_gu.alpha[sl])
        local_dn = ops.GroupedNvfp4Weights.from_checkpoint(w_dn.packed[sl].contiguous(), w_dn.scales_row_major[sl].contiguous(), w_dn.alpha[sl])
        layer, step = parallel.peer_expert_parallel_moe(None, tl, experts, top_k, hidden, inter, local_gu, local_dn)
        ok_peer = True
        x_local, logits_local = xs[rows].contiguous(), logits[rows].contiguous()
        for _ in range(3):
            got = step(x_local, logits_local).clone()
            torch.cuda.synchronize()
            ok_peer = ok_peer and bool(torch.equal(got, ref[rows]))
        layer.barrier.check()
        ok_peer = ok_peer and layer.status() == 0
        result[rank] = (ok_dense, ok_moe, ok_peer)
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
    try:
        for p in procs:
            p.start()
        for p in procs:
            p.join(timeout=300)
    finally:
        for p in procs:  # never leave a worker (and whatever it has on the GPU) behind a failed run
            if p.is_alive():
                p.terminate()
                p.join(timeout=10)
                if p.is_alive():
                    p.kill()
    assert [p.exitcode for p in procs] == [0] * world
    assert dict(result) == {0: (True, True, True), 1: (True, True, True)}


def test_peer_barrier_gives_up_instead_of_spinning():
    # one GPU, two pads: "rank 0" waits for a rank 1 that never signals; the wait must run out, leave a status word and
    # return, and a later barrier that can complete (world of one) must still work on the same context
    torch = pytest.importorskip("torch")
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    import ctypes as C

    from eider_b200 import _lib
    lib = _lib.load()
    words = lib.eider_b200_peer_barrier_pad_bytes() // 4
    pads = [torch.zeros(words, dtype=torch.int32, device="cuda") for _ in range(2)]
    state = torch.zeros(lib.eider_b200_peer_barrier_state_bytes() // 4, dtype=torch.int32, device="cuda")
    table = (C.c_void_p * 2)(*[C.c_void_p(p.data_ptr()) for p in pads])
    assert lib.eider_b200_peer_barrier_on_stream(table, 2, 0, 3, state.data_ptr(), 2_000_000, None) == 0  # ~1 ms budget
    torch.cuda.synchronize()
    status = int(state[-1].item()) & 0xFFFFFFFF
    assert status == (0xBA000000 | (3 << 8) | 1)
    assert int(pads[1][3 * 8 + 0].item()) == 1 and int(pads[0][3 * 8 + 0].item()) == 1  # rank 0 did announce epoch 1
    # the peer arrives late (its flag is set by hand): the next epoch of the same channel completes
    pads[0][3 * 8 + 1] = 2
    state[-1] = 0
    assert lib.eider_b200_peer_barrier_on_stream(table, 2, 0, 3, state.data_ptr(), 2_000_000_000, None) == 0
    torch.cuda.synchronize()
    assert int(state[-1].item()) == 0 and int(state[3].item()) == 2
    assert lib.eider_b200_peer_barrier_on_stream(table, 9, 0, 0, state.data_ptr(), 0, None) == 1
    assert lib.eider_b200_peer_barrier_on_stream(table, 2, 0, 16, state.data_ptr(), 0, None) == 1
