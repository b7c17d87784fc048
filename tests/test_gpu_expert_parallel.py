"""The expert-parallel routed-MoE layer with device-resident counts, with several ranks emulated on ONE GPU: every
"rank" is an instance with its own buffers, the pointer tables hold all instances' buffers, and the phases run rank
after rank, which satisfies every barrier of the real layer by stream order.  The result must equal the single-GPU
pipeline bit for bit (rows of an expert arrive in global route order, so every GEMM row sees the same operands)."""
import numpy as np
import pytest

from tests.util import require_cuda

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("world,tokens,experts,top_k,hidden,inter", [(2, 64, 8, 2, 256, 128), (4, 512, 16, 4, 1024, 384),
                                                                      (8, 96, 128, 8, 256, 128)])
def test_emulated_ranks_equal_single_gpu(world, tokens, experts, top_k, hidden, inter):
    torch = require_cuda()
    from eider_b200 import ops, parallel
    g = torch.Generator(device="cuda").manual_seed(world * 100 + tokens)
    x = torch.randn(tokens, hidden, device="cuda", generator=g).to(torch.bfloat16)
    logits = torch.randn(tokens, experts, device="cuda", generator=g)
    if world == 8:
        logits[:, 5] += 4.0  # a hot expert and many empty ones: ragged counts, ranks that receive almost nothing
    w_gu = ops.GroupedNvfp4Weights.quantize(torch.randn(experts, 2 * inter, hidden, device="cuda", generator=g) * 0.02)
    w_dn = ops.GroupedNvfp4Weights.quantize(torch.randn(experts, hidden, inter, device="cuda", generator=g) * 0.02)
    ref = ops.GroupedMoe(tokens, experts, top_k, hidden, inter).run(x, logits, w_gu, w_dn).clone()

    per, tl = experts // world, tokens // world
    ranks = []
    for r in range(world):
        sl = slice(r * per, (r + 1) * per)
        gu = ops.GroupedNvfp4Weights.from_checkpoint(w_gu.packed[sl].contiguous(), w_gu.scales_row_major[sl].contiguous(), w_gu.alpha[sl])
        dn = ops.GroupedNvfp4Weights.from_checkpoint(w_dn.packed[sl].contiguous(), w_dn.scales_row_major[sl].contiguous(), w_dn.alpha[sl])
        ranks.append(parallel.PeerExpertParallelMoe(r, world, tl, experts, top_k, hidden, inter, gu, dn))
    pointers = {name: [rk.buffers[name].data_ptr() for rk in ranks] for name in parallel.PeerExpertParallelMoe.PEER_BUFFERS}
    for rk in ranks:
        rk.connect(pointers)
    for step in range(2):  # the second step reuses every buffer
        for r, rk in enumerate(ranks):
            rk.route_and_publish(x[r * tl:(r + 1) * tl].contiguous(), logits[r * tl:(r + 1) * tl].contiguous())
        for rk in ranks:
            rk.dispatch()
        for rk in ranks:
            rk.run_experts_and_return()
        out = torch.cat([rk.combine() for rk in ranks])
        torch.cuda.synchronize()
        assert all(rk.status() == 0 for rk in ranks)
        assert sum(int(rk.recv_total.item()) for rk in ranks) == tokens * top_k
        assert torch.equal(out, ref)
