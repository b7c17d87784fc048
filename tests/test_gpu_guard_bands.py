"""Guard bands: every output buffer of a call is followed (and preceded) by poison bytes that must survive the call, and
outputs start poisoned so that an element the kernel skips shows up.  Stands in for a memory checker on the kernels whose
index arithmetic is the least trivial: ragged quantizer rows, per-expert scale tiles, partial GEMM tiles, split-K decode."""
import numpy as np
import pytest

from tests.util import require_cuda

pytestmark = pytest.mark.gpu
GUARD = 256


def guarded(torch, nbytes, dtype, fill=0xAB):
    """-> (view of `nbytes` bytes as dtype, checker) inside a buffer with GUARD poison bytes on both sides."""
    raw = torch.full((nbytes + 2 * GUARD,), fill, dtype=torch.uint8, device="cuda")
    body = raw[GUARD:GUARD + nbytes].view(dtype)

    def intact():
        return bool((raw[:GUARD] == fill).all().item()) and bool((raw[GUARD + nbytes:] == fill).all().item())

    return body, intact


def test_quantizers_stay_inside_their_outputs():
    torch = require_cuda()
    from eider_b200 import _lib, ops
    lib = _lib.load()
    for tokens, k in [(3, 96), (130, 2064), (512, 5120), (1, 16)]:
        x = torch.randn(tokens, k, device="cuda")
        xb = x.to(torch.bfloat16)
        n_sf = ops.scale_layout_len(tokens, k)
        for name, src, args in (("infer_quantize_nvfp4_col_major_f32_on_stream", x, (0.5,)),
                                ("eider_b200_quantize_nvfp4_bf16_on_stream", xb, (0.5,))):
            packed, ok_p = guarded(torch, tokens * k // 2, torch.uint8)
            scales, ok_s = guarded(torch, n_sf, torch.uint8)
            assert getattr(lib, name)(src.data_ptr(), packed.data_ptr(), scales.data_ptr(), k, tokens, *args, None) == 0
            torch.cuda.synchronize()
            assert ok_p() and ok_s(), (name, tokens, k)
        packed, ok_p = guarded(torch, tokens * k // 2, torch.uint8)
        scales, ok_s = guarded(torch, n_sf, torch.uint8)
        rows, ok_r = guarded(torch, tokens * 4, torch.float32)
        assert lib.eider_b200_quantize_nvfp4_rowscale_on_stream(xb.data_ptr(), 1, packed.data_ptr(), scales.data_ptr(), rows.data_ptr(), k,
                                                                tokens, None) == 0
        torch.cuda.synchronize()
        assert ok_p() and ok_s() and ok_r(), (tokens, k)
        assert not bool((packed == 0xAB).all().item())


# (the last two: K split over three work items per tile, fp32 partial sums summed by the reduce kernel)
@pytest.mark.parametrize("m,n,k,block_n,splits", [(130, 264, 1056, 0, 0), (300, 328, 512, 512, 0), (512, 1024, 1024, 512, 0), (1, 144, 64, 0, 0),
                                                  (100, 330, 4096, 128, 3), (300, 328, 3072, 512, 3), (300, 328, 512, 384, 0), (260, 1000, 1024, 384, 2)])
def test_dense_gemm_writes_exactly_its_output(m, n, k, block_n, splits):
    torch = require_cuda()
    from eider_b200 import ops
    w = ops.ModelOptWeight.quantize(torch.randn(n, k, device="cuda") * 0.02)
    xq = ops.quantize_nvfp4_rowscale(torch.randn(m, k, device="cuda").to(torch.bfloat16))
    for dtype, size in ((torch.bfloat16, 2), (torch.float32, 4)):
        body, intact = guarded(torch, m * n * size, dtype, fill=0xFF)  # 0xFF.. is NaN in both types
        out = body.view(m, n)
        plan = ops.Fp4TnMatmulPlan(m, n, k)
        if block_n:
            plan.set_block_n(block_n)
        if splits:
            plan.set_k_splits(splits)
        plan.run(xq, w, out=out)
        torch.cuda.synchronize()
        assert plan.status() == 0 and intact()
        assert not torch.isnan(out.float()).any()  # every element was written


def test_moe_rows_and_grouped_gemm_stay_inside():
    torch = require_cuda()
    from eider_b200 import _lib, ops
    lib = _lib.load()
    tokens, experts, top_k, hidden, inter = 70, 6, 3, 256, 128
    routes = tokens * top_k
    x = torch.randn(tokens, hidden, device="cuda").to(torch.bfloat16)
    idx = torch.randint(0, experts, (routes,), dtype=torch.int32, device="cuda")
    idx[idx == 2] = 3  # an empty expert in the middle
    r = ops.MoeSortedRoutes(routes, experts).sort(idx)
    tile = ops.moe_scale_tile_bytes(hidden)
    packed, ok_p = guarded(torch, routes * hidden // 2, torch.uint8)
    scales, ok_s = guarded(torch, ((routes + 127) // 128 + experts) * tile, torch.uint8)
    src_p = torch.zeros(tokens, hidden // 2, dtype=torch.uint8, device="cuda")
    src_s = torch.zeros(ops.scale_layout_len(tokens, hidden), dtype=torch.uint8, device="cuda")
    assert lib.eider_b200_moe_gather_quantize_sorted_routes_nvfp4_bf16_on_stream(
        x.data_ptr(), r.sorted_routes.data_ptr(), r.sorted_experts.data_ptr(), r.expert_offsets.data_ptr(), src_p.data_ptr(), src_s.data_ptr(),
        packed.data_ptr(), scales.data_ptr(), tokens, routes, top_k, hidden, tile, None) == 0
    w = ops.GroupedNvfp4Weights.quantize(torch.randn(experts, 2 * inter, hidden, device="cuda") * 0.02)
    out, ok_o = guarded(torch, routes * 2 * inter * 2, torch.bfloat16, fill=0xFF)
    plan = ops.Fp4GroupedGemmPlan(2 * inter, tokens, hidden, experts)
    assert lib.eider_b200_nvfp4_grouped_gemm_on_stream(plan._plan, packed.data_ptr(), scales.data_ptr(), w.packed.data_ptr(),
                                                       w.scales_tiled.data_ptr(), out.data_ptr(), w.alpha.data_ptr(),
                                                       r.expert_offsets.data_ptr(), routes, None) == 0
    # the fused SiLU epilogue writes the down projection's input and nothing else
    wi = w.interleave_gate_up()
    tile_i = ops.moe_scale_tile_bytes(inter)
    act_p, ok_ap = guarded(torch, routes * inter // 2, torch.uint8)
    act_s, ok_as = guarded(torch, ((routes + 127) // 128 + experts) * tile_i, torch.uint8)
    assert lib.eider_b200_nvfp4_grouped_gemm_silu_quantize_on_stream(plan._plan, packed.data_ptr(), scales.data_ptr(), wi.packed.data_ptr(),
                                                                     wi.scales_tiled.data_ptr(), wi.alpha.data_ptr(),
                                                                     r.expert_offsets.data_ptr(), routes, act_p.data_ptr(), act_s.data_ptr(),
                                                                     tile_i, None) == 0
    torch.cuda.synchronize()
    assert plan.status() == 0
    assert ok_p() and ok_s() and ok_o() and ok_ap() and ok_as()
    assert not torch.isnan(out.view(routes, 2 * inter).float()).any()


@pytest.mark.parametrize("tokens,n,k", [(1, 13824, 5120), (3, 1000, 2048), (40, 520, 1024)])
def test_decode_writes_exactly_its_output(tokens, n, k):
    torch = require_cuda()
    from eider_b200 import ops
    w = ops.ModelOptWeight.quantize(torch.randn(n, k, device="cuda") * 0.02)
    x = torch.randn(tokens, k, device="cuda").to(torch.bfloat16)
    body, intact = guarded(torch, tokens * n * 2, torch.bfloat16, fill=0xFF)
    plan = ops.Nvfp4DecodePlan(64, n, k)
    plan.run(x, w, out=body.view(tokens, n))
    torch.cuda.synchronize()
    assert plan.status() == 0 and intact()
    assert not torch.isnan(body.float()).any()
