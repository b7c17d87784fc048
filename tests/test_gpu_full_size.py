"""Parity at the sizes the benchmark numbers are quoted on.

The dense prefill GEMM (512 x 5120 x 27648, CTA-pair kernel, per-row-scale quantizer, bf16 output) is compared with the
oracle on every output element; the larger chunks of the sweep (2048 and 16384 tokens, and the down projection
13824 -> 5120) on column slabs that contain the first, a middle and the last weight tile; the routed-MoE layer (4096
tokens, 128 experts, top-8, hidden 2048, intermediate 768) bit-exactly on router, permutation and gather + quantize,
and on sampled experts (first, last, fullest, emptiest) x column slabs for the two grouped GEMMs, with the combine on
every token.  The criterion is the reference's: GPU result against host dequantize + fp32-accumulated matmul
(crates/eider-cuda/src/cublaslt/fp4_tn.rs:1503-1542; crates/eider-cuda/benches/qwen38_grouped_moe_prefill.rs:272-306).
Weights are quantized on the device (that quantizer is held bit-exact to the oracle in test_gpu_quantize.py) and the
oracle dequantizes the same bytes."""
import numpy as np
import pytest

from tests.util import gemm_close, require_cuda, to_np

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    require_cuda()
    from eider_b200 import ops
    return ops


def _dense_case(ops, oracle, m, k, n, slabs, seed):
    """slabs: list of (first column, width) to compare, or None for every column."""
    import torch
    g = torch.Generator(device="cuda").manual_seed(seed)
    w = torch.randn(n, k, device="cuda", generator=g) * 0.02
    wd = ops.ModelOptWeight.quantize(w)
    del w
    x = torch.randn(m, k, device="cuda", generator=g).to(torch.bfloat16)
    xq = ops.quantize_nvfp4_rowscale(x)
    plan = ops.Fp4TnMatmulPlan(m, n, k)
    y = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")  # poison: every element must be written
    plan.run(xq, wd, out=y)
    torch.cuda.synchronize()
    assert plan.status() == 0
    # the activation quantizer, bit for bit, at this size
    xp, xs, xr = oracle.quantize_nvfp4_rowscale(x.float().cpu().numpy())
    assert np.array_equal(xq.packed.cpu().numpy(), xp)
    assert np.array_equal(xq.scales.cpu().numpy(), xs)
    assert np.array_equal(xq.row_scales.cpu().numpy(), xr)
    a = oracle.dequantize_tiled(xp, xs)
    wp, ws = wd.packed.cpu().numpy(), wd.scales_row_major.cpu().numpy()
    checked = 0
    worst = 0.0
    for c0, width in (slabs or [(0, n)]):
        ref = oracle.matmul_nt(a, oracle.dequantize_weight(wp[c0:c0 + width], ws[c0:c0 + width]), alpha=wd.weight_scale_2, row_scale=xr)
        got = to_np(y[:, c0:c0 + width])
        assert not np.isnan(got).any()
        ok, stats = gemm_close(got, ref)
        assert ok, (c0, stats)
        checked += got.size
        worst = max(worst, stats["max_rel_err_over_floor"])
    assert not torch.isnan(y.float()).any()
    return plan.block_n, checked, worst


def test_prefill_gemm_headline_shape_every_element(ops, oracle):
    block_n, checked, worst = _dense_case(ops, oracle, 512, 5120, 27648, None, seed=0)
    assert block_n == 512  # the CTA-pair kernel is what this shape runs
    assert checked == 512 * 27648 and worst <= 1e-2


@pytest.mark.parametrize("m", [128, 2048, 16384])
def test_prefill_gemm_sweep_gate_up(ops, oracle, m):
    n = 27648
    _dense_case(ops, oracle, m, 5120, n, [(0, 256), (n // 2 - 128, 256), (n - 256, 256)], seed=m)


@pytest.mark.parametrize("m", [512, 2048, 8192])
def test_prefill_gemm_sweep_down_projection(ops, oracle, m):
    n = 5120
    _dense_case(ops, oracle, m, 13824, n, [(0, 256), (n // 2 - 128, 256), (n - 256, 256)], seed=m + 1)


def _u32(t):
    return t.cpu().numpy().view(np.uint32)


def test_routed_moe_benchmark_size(ops, oracle):
    import torch
    tokens, experts, top_k, hidden, inter = 4096, 128, 8, 2048, 768
    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randn(tokens, hidden, device="cuda", generator=g).to(torch.bfloat16)
    logits = torch.randn(tokens, experts, device="cuda", generator=g)
    w_gu = ops.GroupedNvfp4Weights.quantize(torch.randn(experts, 2 * inter, hidden, device="cuda", generator=g) * 0.02)
    w_dn = ops.GroupedNvfp4Weights.quantize(torch.randn(experts, hidden, inter, device="cuda", generator=g) * 0.02)
    moe = ops.GroupedMoe(tokens, experts, top_k, hidden, inter)
    out = moe.run(x, logits, w_gu, w_dn)
    torch.cuda.synchronize()
    assert moe.gate_up_plan.status() == 0 and moe.down_plan.status() == 0

    # router, permutation, gather + quantize: every byte
    xh = x.float().cpu().numpy()
    idx, w = oracle.moe_topk(logits.cpu().numpy(), top_k, True)
    assert np.array_equal(_u32(moe.route_indices), idx)
    assert np.allclose(moe.route_weights.cpu().numpy(), w, rtol=1e-5, atol=1e-7)
    counts, offsets, sorted_routes, sorted_experts, inverse = oracle.moe_sort_routes(idx.reshape(-1), experts)
    r = moe.routes
    assert np.array_equal(_u32(r.expert_counts), counts) and np.array_equal(_u32(r.expert_offsets), offsets)
    assert np.array_equal(_u32(r.sorted_routes), sorted_routes) and np.array_equal(_u32(r.route_to_sorted), inverse)
    a_p, a_s = oracle.moe_gather_quantize(xh, sorted_routes, sorted_experts, offsets, top_k, experts)
    assert np.array_equal(moe.gate_up_in.packed.cpu().numpy(), a_p)
    assert np.array_equal(moe.gate_up_in.scales.cpu().numpy(), a_s)

    # grouped GEMMs on sampled experts x column slabs, each stage fed with the device's own input bytes
    sample = sorted({0, experts - 1, int(np.argmax(counts)), int(np.argmin(counts))})
    d_p, d_s = moe.down_in.packed.cpu().numpy(), moe.down_in.scales.cpu().numpy()
    gu_out = moe.gate_up_out.view(torch.int16).cpu().numpy().view(np.uint16)
    dn_out = moe.down_out.view(torch.int16).cpu().numpy().view(np.uint16)
    # SiLU * up + quantize from the device's gate/up rows (expf differs in the last place between device and host)
    s_p, s_s = oracle.moe_silu_mul_quantize(gu_out, sorted_experts, offsets, experts)
    assert np.count_nonzero(d_p != s_p) / d_p.size < 2e-3
    assert np.count_nonzero(d_s != s_s) / d_s.size < 2e-3

    def expert_rows(packed, scales, e, k):
        r0, r1 = int(offsets[e]), int(offsets[e + 1])
        base = oracle.moe_scale_base(e, offsets, oracle.moe_scale_tile_bytes(k))
        return r0, r1, oracle.dequantize_tiled(packed[r0:r1], scales[base: base + oracle.scale_layout_len(r1 - r0, k)])

    checked = 0
    for e in sample:
        if counts[e] == 0:
            continue
        for (weights, in_p, in_s, k, n, got_bits) in ((w_gu, a_p, a_s, hidden, 2 * inter, gu_out), (w_dn, d_p, d_s, inter, hidden, dn_out)):
            r0, r1, act = expert_rows(in_p, in_s, e, k)
            wp = weights.packed[e].cpu().numpy()
            wsr = weights.scales_row_major[e].cpu().numpy()
            alpha = float(weights.alpha[e].item())
            for c0 in (0, n - 256):
                ref = oracle.bf16_round(oracle.matmul_nt(act, oracle.dequantize_weight(wp[c0:c0 + 256], wsr[c0:c0 + 256]), alpha=alpha))
                got = oracle.bf16_bits_to_f32(got_bits[r0:r1, c0:c0 + 256])
                ok, stats = gemm_close(got, ref)
                assert ok, (e, k, c0, stats)
                checked += got.size
    assert checked > 0
    # weighted un-permute of the device's down rows: every token
    ref = oracle.moe_combine(inverse, w.reshape(-1), dn_out, tokens, top_k)
    assert np.allclose(out.cpu().numpy(), ref, rtol=1e-5, atol=1e-6)
