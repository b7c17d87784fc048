"""Routed-MoE pipeline against the oracle: router, permutation (bit-exact), gather + quantize (bit-exact),
grouped GEMM, SiLU * up + quantize, combine, and the whole pipeline at reduced sizes (the benchmark size is in
test_gpu_full_size.py)."""
import numpy as np
import pytest

from tests.util import gemm_close, require_cuda, to_np

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    require_cuda()
    from eider_b200 import ops
    return ops


def _dev(a, dtype=None):
    import torch
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    return t if dtype is None else t.to(dtype)


def _i32(a):
    return _dev(np.ascontiguousarray(a, np.uint32).view(np.int32))


def _u32(t):
    return t.cpu().numpy().view(np.uint32)


def test_router_golden(ops):
    # crates/eider-cuda/src/kernels/non_gemm.rs:17752-17809 and :17935-17959
    lg = np.array([[0.0, 3.0, 1.0, 2.0]], np.float32)
    for norm in (True, False):
        idx, w = ops.moe_topk(_dev(lg), 2, norm)
        assert _u32(idx).tolist() == [[1, 3]]
        if norm:
            assert abs(float(w.sum()) - 1.0) < 1e-6
        else:
            p = np.exp(lg - lg.max())
            p /= p.sum()
            assert np.allclose(w.cpu().numpy()[0], p[0, [1, 3]], atol=1e-6)
    lg = np.full((1, 256), -10.0, np.float32)
    for e in [19, 3, 241, 7, 8, 9, 10, 11, 12]:
        lg[0, e] = 4.0
    idx, w = ops.moe_topk(_dev(lg), 8, True)
    assert _u32(idx).tolist() == [[3, 7, 8, 9, 10, 11, 12, 19]]
    assert np.allclose(w.cpu().numpy(), 0.125)
    lg = np.full((2, 8), np.nan, np.float32)
    for norm in (True, False):
        idx, w = ops.moe_topk(_dev(lg), 3, norm)
        assert _u32(idx).tolist() == [[0, 1, 2], [0, 1, 2]]
        assert w.cpu().numpy().tolist() == [[1.0, 0.0, 0.0]] * 2


@pytest.mark.parametrize("tokens,experts,k", [(37, 128, 8), (4096, 128, 8), (64, 512, 10), (9, 60, 4)])
@pytest.mark.parametrize("norm", [True, False])
def test_router_random(ops, oracle, tokens, experts, k, norm):
    rng = np.random.default_rng(tokens + experts)
    lg = rng.standard_normal((tokens, experts)).astype(np.float32)
    lg[0, :3] = [np.inf, np.nan, -np.inf]
    idx, w = ops.moe_topk(_dev(lg), k, norm)
    oi, ow = oracle.moe_topk(lg, k, norm)
    assert np.array_equal(_u32(idx), oi)
    assert np.allclose(w.cpu().numpy(), ow, rtol=1e-5, atol=1e-7)


def test_permute_golden(ops):
    # crates/eider-cuda/src/kernels/non_gemm.rs:15780-15817
    ind = np.array([3, 1, 3, 0, 1, 2, 3, 2], np.uint32)
    r = ops.MoeSortedRoutes(8, 4).sort(_i32(ind))
    assert _u32(r.expert_counts).tolist() == [1, 2, 2, 3]
    assert _u32(r.expert_offsets).tolist() == [0, 1, 3, 5, 8]
    assert _u32(r.sorted_experts).tolist() == [0, 1, 1, 2, 2, 3, 3, 3]
    inv, sr = _u32(r.route_to_sorted), _u32(r.sorted_routes)
    for i in range(8):
        assert sr[inv[i]] == i


@pytest.mark.parametrize("routes,experts", [(1, 1), (300, 5), (32768, 128), (5000, 1000)])
def test_permute_matches_oracle(ops, oracle, routes, experts):
    rng = np.random.default_rng(routes)
    ind = rng.integers(0, experts, routes).astype(np.uint32)
    r = ops.MoeSortedRoutes(routes, experts).sort(_i32(ind))
    counts, offsets, sorted_routes, sorted_experts, inverse = oracle.moe_sort_routes(ind, experts)
    assert np.array_equal(_u32(r.expert_counts), counts)
    assert np.array_equal(_u32(r.expert_offsets), offsets)
    assert np.array_equal(_u32(r.sorted_routes), sorted_routes)  # stable: ascending route order inside an expert
    assert np.array_equal(_u32(r.sorted_experts), sorted_experts)
    assert np.array_equal(_u32(r.route_to_sorted), inverse)


def test_gather_quantize_matches_oracle(ops, oracle):
    # calibrated fixture shape of crates/eider-cuda/src/kernels/non_gemm.rs:15168-15249: 7 tokens x top-3 x 5 experts x K=80
    tokens, k_, experts, feat = 7, 3, 5, 80
    rng = np.random.default_rng(0)
    x = rng.standard_normal((tokens, feat)).astype(np.float32)
    ind = np.array([[0, 4, 1], [0, 1, 4], [3, 0, 2], [1, 2, 3], [4, 3, 0], [2, 1, 0], [3, 4, 2]], np.uint32).reshape(-1)
    r = ops.MoeSortedRoutes(tokens * k_, experts).sort(_i32(ind))
    rows = ops.MoeSortedNvfp4Rows(tokens * k_, experts, feat, tokens).gather_quantize(_dev(x), r, k_)
    counts, offsets, sorted_routes, sorted_experts, inverse = oracle.moe_sort_routes(ind, experts)
    packed, scales = oracle.moe_gather_quantize(x, sorted_routes, sorted_experts, offsets, k_, experts)
    assert np.array_equal(rows.packed.cpu().numpy(), packed)
    assert np.array_equal(rows.scales.cpu().numpy(), scales)


def test_combine_golden_with_guard(ops, oracle):
    # crates/eider-cuda/src/kernels/non_gemm.rs:15821-15887 incl. the guard elements after the output
    import torch
    for ln in (5, 6, 16):
        rows, k = 2, 2
        inverse = np.array([1, 0, 3, 2], np.uint32)
        weights = np.array([0.25, 0.75, 0.4, 0.6], np.float32)
        src = oracle.f32_to_bf16_bits(((np.arange(4 * ln) - 7) / 8.0).astype(np.float32)).reshape(4, ln)
        r = ops.MoeSortedRoutes(4, 2)
        r.route_to_sorted.copy_(_i32(inverse))
        buf = torch.full((rows * ln + 7,), -77.0, dtype=torch.float32, device="cuda")
        ops.moe_weighted_accumulate(r, _dev(weights), _dev(src.view(np.int16)).view(torch.bfloat16), rows, k,
                                    out=buf[: rows * ln].view(rows, ln))
        got = buf.cpu().numpy()
        assert np.all(got[rows * ln:] == -77.0)
        assert np.allclose(got[: rows * ln].reshape(rows, ln), oracle.moe_combine(inverse, weights, src, rows, k), atol=1e-6)


def _pipeline(ops, oracle, tokens, experts, top_k, hidden, inter, seed, check_stages=True):
    import torch
    rng = np.random.default_rng(seed)
    x = oracle.bf16_round(rng.standard_normal((tokens, hidden)).astype(np.float32))
    logits = rng.standard_normal((tokens, experts)).astype(np.float32)
    wgu = (rng.standard_normal((experts, 2 * inter, hidden)) * 0.02).astype(np.float32)
    wdn = (rng.standard_normal((experts, hidden, inter)) * 0.02).astype(np.float32)
    q = [oracle.quantize_weight(wgu[e]) for e in range(experts)]
    gu_p, gu_s, gu_a = np.stack([a[0] for a in q]), np.stack([a[1] for a in q]), np.array([a[2] for a in q], np.float32)
    q = [oracle.quantize_weight(wdn[e]) for e in range(experts)]
    dn_p, dn_s, dn_a = np.stack([a[0] for a in q]), np.stack([a[1] for a in q]), np.array([a[2] for a in q], np.float32)
    w_gu = ops.GroupedNvfp4Weights.from_checkpoint(_dev(gu_p), _dev(gu_s), _dev(gu_a))
    w_dn = ops.GroupedNvfp4Weights.from_checkpoint(_dev(dn_p), _dev(dn_s), _dev(dn_a))
    moe = ops.GroupedMoe(tokens, experts, top_k, hidden, inter)
    out = moe.run(_dev(x, torch.bfloat16), _dev(logits), w_gu, w_dn)
    torch.cuda.synchronize()
    assert moe.gate_up_plan.status() == 0 and moe.down_plan.status() == 0

    # oracle, stage by stage
    idx, w = oracle.moe_topk(logits, top_k, True)
    counts, offsets, sorted_routes, sorted_experts, inverse = oracle.moe_sort_routes(idx.reshape(-1), experts)
    a_p, a_s = oracle.moe_gather_quantize(x, sorted_routes, sorted_experts, offsets, top_k, experts)
    gate_up = oracle.moe_grouped_gemm(a_p, a_s, offsets, gu_p, gu_s, gu_a)
    if check_stages:
        assert np.array_equal(_u32(moe.route_indices), idx)
        assert np.array_equal(moe.gate_up_in.packed.cpu().numpy(), a_p)
        assert np.array_equal(moe.gate_up_in.scales.cpu().numpy(), a_s)
        ok, stats = gemm_close(to_np(moe.gate_up_out), oracle.bf16_bits_to_f32(gate_up))
        assert ok, stats
    # continue the oracle from the device's gate/up rows so the SiLU stage is compared on identical inputs
    dev_gu_bits = moe.gate_up_out.view(torch.int16).cpu().numpy().view(np.uint16)
    d_p, d_s, act = oracle.moe_silu_mul_quantize(dev_gu_bits, sorted_experts, offsets, experts, want_act=True)
    if check_stages:
        got_p = moe.down_in.packed.cpu().numpy()
        mism = np.count_nonzero(got_p != d_p) / got_p.size
        assert mism < 2e-3, mism  # expf differs in the last ulp between device and host
        deq_dev = _deq_rows(oracle, got_p, moe.down_in.scales.cpu().numpy(), offsets, inter)
        assert np.all(np.abs(deq_dev - act) <= 0.27 * np.abs(act).reshape(act.shape[0], -1, 16).max(axis=2).repeat(16, axis=1) + 1e-12)
    dev_dp, dev_ds = moe.down_in.packed.cpu().numpy(), moe.down_in.scales.cpu().numpy()
    down = oracle.moe_grouped_gemm(dev_dp, dev_ds, offsets, dn_p, dn_s, dn_a)
    ok, stats = gemm_close(to_np(moe.down_out), oracle.bf16_bits_to_f32(down))
    assert ok, stats
    dev_down_bits = moe.down_out.view(torch.int16).cpu().numpy().view(np.uint16)
    ref = oracle.moe_combine(inverse, w.reshape(-1), dev_down_bits, tokens, top_k)
    assert np.allclose(out.cpu().numpy(), ref, rtol=1e-5, atol=1e-6)
    # end to end against the all-oracle pipeline
    d_p2, d_s2 = oracle.moe_silu_mul_quantize(gate_up, sorted_experts, offsets, experts)
    down2 = oracle.moe_grouped_gemm(d_p2, d_s2, offsets, dn_p, dn_s, dn_a)
    ref2 = oracle.moe_combine(inverse, w.reshape(-1), down2, tokens, top_k)
    ok, stats = gemm_close(out.cpu().numpy(), ref2, rel=3e-2, abs_frac=3e-2)
    assert ok, stats


def _deq_rows(oracle, packed, scales, offsets, k):
    out = np.zeros((packed.shape[0], k), np.float32)
    tile = oracle.moe_scale_tile_bytes(k)
    for e in range(len(offsets) - 1):
        r0, r1 = int(offsets[e]), int(offsets[e + 1])
        if r0 == r1:
            continue
        base = oracle.moe_scale_base(e, offsets, tile)
        n = r1 - r0
        out[r0:r1] = oracle.dequantize_tiled(packed[r0:r1], scales[base: base + oracle.scale_layout_len(n, k)])
    return out


def test_pipeline_small(ops, oracle):
    _pipeline(ops, oracle, tokens=96, experts=8, top_k=2, hidden=256, inter=128, seed=1)


def test_pipeline_ragged_experts(ops, oracle):
    # more experts than routes: many empty experts, partial 128-row tiles
    _pipeline(ops, oracle, tokens=20, experts=16, top_k=3, hidden=512, inter=128, seed=2)


def test_pipeline_medium(ops, oracle):
    _pipeline(ops, oracle, tokens=512, experts=16, top_k=4, hidden=1024, inter=384, seed=3)


@pytest.mark.parametrize("tokens,experts,top_k,hidden,inter", [(96, 8, 2, 256, 128), (20, 16, 3, 512, 128), (512, 16, 4, 1024, 384),
                                                               (2048, 128, 8, 2048, 768)])
def test_fused_silu_epilogue_equals_staged_pipeline(ops, tokens, experts, top_k, hidden, inter):
    # the gate/up grouped GEMM with SiLU * up -> NVFP4 in its epilogue against the GEMM + stand-alone quantizer: the down
    # projection's input must be the same bytes (ragged and empty experts included), hence the same layer output
    import torch
    g = torch.Generator(device="cuda").manual_seed(tokens + experts)
    x = torch.randn(tokens, hidden, device="cuda", generator=g).to(torch.bfloat16)
    logits = torch.randn(tokens, experts, device="cuda", generator=g)
    w_gu = ops.GroupedNvfp4Weights.quantize(torch.randn(experts, 2 * inter, hidden, device="cuda", generator=g) * 0.02)
    w_dn = ops.GroupedNvfp4Weights.quantize(torch.randn(experts, hidden, inter, device="cuda", generator=g) * 0.02)
    staged = ops.GroupedMoe(tokens, experts, top_k, hidden, inter)
    ref = staged.run(x, logits, w_gu, w_dn).clone()
    fused = ops.GroupedMoe(tokens, experts, top_k, hidden, inter)
    out = fused.run(x, logits, w_gu, w_dn, w_gate_up_interleaved=w_gu.interleave_gate_up())
    torch.cuda.synchronize()
    assert fused.gate_up_plan.status() == 0 and fused.down_plan.status() == 0
    assert torch.equal(fused.down_in.packed, staged.down_in.packed)
    # scale bytes: compare what belongs to routes (padding rows of the per-expert tiles are never written by either path)
    offsets = staged.routes.expert_offsets.cpu().numpy().view(np.uint32)
    fs, ss = fused.down_in.scales.cpu().numpy(), staged.down_in.scales.cpu().numpy()
    tile = staged.down_in.tile_bytes
    blocks = inter // 16
    for e in range(experts):
        n = int(offsets[e + 1] - offsets[e])
        if n == 0:
            continue
        base = ((int(offsets[e]) + 127) // 128 + e) * tile
        rows_ = np.arange(n)[:, None]
        kb = np.arange(blocks)[None, :]
        padded = (blocks + 3) // 4 * 4
        off = base + ((kb // 4) * 4 + (rows_ // 128) * padded) * 128 + (rows_ % 32) * 16 + ((rows_ % 128) // 32) * 4 + kb % 4
        assert np.array_equal(fs[off], ss[off]), e
    assert torch.equal(out, ref)
