"""Decode-side routed MoE and the lm-head arg-max through the reference's entry points (device pointer tables), against
a host evaluation of the same dequantized operands (crates/eider-cuda/src/format.rs:379-392 semantics: dequantize, f32
products, the sum order is free)."""
import numpy as np
import pytest

from tests.util import gemm_close, require_cuda

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def lib():
    require_cuda()
    from eider_b200 import _lib
    return _lib.load()


def dev(a, dtype=None):
    import torch
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    return t if dtype is None else t.to(dtype)


def table(tensors):
    import torch
    return torch.tensor([t.data_ptr() for t in tensors], dtype=torch.int64, device="cuda")


def make_experts(oracle, rng, experts, n, k):
    """-> host (packed, scales, global) per expert and the dequantized f64 matrices."""
    out = []
    for _ in range(experts):
        w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
        p, s, g = oracle.quantize_weight(w)
        out.append((p, s, float(g), oracle.dequantize_weight(p, s).astype(np.float64) * float(g)))
    return out


@pytest.mark.parametrize("tokens", [1, 3])
def test_decode_moe_layer(lib, oracle, tokens):
    # one decode step of a routed layer: router -> grouped gate/up GEMV -> SiLU * up per slot -> grouped down GEMV over
    # per-slot inputs -> weighted accumulation + shared expert + residual (rounded to bf16 precision)
    import torch
    experts, top_k, hidden, inter = 16, 4, 512, 256
    rng = np.random.default_rng(tokens)
    gu = make_experts(oracle, rng, experts, 2 * inter, hidden)
    dn = make_experts(oracle, rng, experts, hidden, inter)
    gu_dev = [(dev(p), dev(s)) for p, s, _, _ in gu]
    dn_dev = [(dev(p), dev(s)) for p, s, _, _ in dn]
    gu_w, gu_s, gu_g = table([a for a, _ in gu_dev]), table([b for _, b in gu_dev]), dev(np.array([g for _, _, g, _ in gu], np.float32))
    dn_w, dn_s, dn_g = table([a for a, _ in dn_dev]), table([b for _, b in dn_dev]), dev(np.array([g for _, _, g, _ in dn], np.float32))
    ones = torch.ones(experts, device="cuda")
    x = rng.standard_normal((tokens, hidden)).astype(np.float32)
    logits = rng.standard_normal((tokens, experts)).astype(np.float32)
    shared_out = rng.standard_normal((tokens, hidden)).astype(np.float32)
    shared_logit = rng.standard_normal(tokens).astype(np.float32)
    residual = rng.standard_normal((tokens, hidden)).astype(np.float32)
    xd, ld = dev(x), dev(logits)
    idx = torch.zeros(tokens, top_k, dtype=torch.int32, device="cuda")
    wts = torch.zeros(tokens, top_k, device="cuda")
    assert lib.infer_moe_topk_f32_batch_on_stream(ld.data_ptr(), idx.data_ptr(), wts.data_ptr(), tokens, experts, top_k, 1, None) == 0
    routes = tokens * top_k
    gate_up = torch.zeros(routes, 2 * inter, device="cuda")
    act = torch.zeros(routes, inter, device="cuda")
    down = torch.zeros(routes, hidden, device="cuda")
    gate_up_t, act_t, down_t = table(list(gate_up)), table(list(act)), table(list(down))
    out = torch.zeros(tokens, hidden, device="cuda")
    for t in range(tokens):  # the shared-input GEMV takes one token's slots at a time
        assert lib.infer_nvfp4_w4a16_grouped_matvec_f32_on_stream(
            idx[t].data_ptr(), xd[t].data_ptr(), gu_w.data_ptr(), gu_s.data_ptr(), gu_g.data_ptr(), gate_up_t[t * top_k:].data_ptr(),
            experts, top_k, 2 * inter, hidden, None) == 0
    assert lib.infer_moe_silu_slots_f32_on_stream(idx.data_ptr(), gate_up_t.data_ptr(), act_t.data_ptr(), ones.data_ptr(), inter, routes, None) == 0
    assert lib.infer_nvfp4_w4a16_grouped_inputs_matvec_f32_on_stream(idx.data_ptr(), act_t.data_ptr(), dn_w.data_ptr(), dn_s.data_ptr(),
                                                                     dn_g.data_ptr(), down_t.data_ptr(), experts, routes, hidden, inter, None) == 0
    sd, sld, rd = dev(shared_out), dev(shared_logit), dev(residual)
    assert lib.infer_qwen36_ffn_finalize_routed_batch_f32_on_stream(idx.data_ptr(), wts.data_ptr(), down_t.data_ptr(), ones.data_ptr(),
                                                                    sld.data_ptr(), sd.data_ptr(), rd.data_ptr(), out.data_ptr(), tokens,
                                                                    hidden, top_k, None) == 0
    acc = torch.zeros(tokens, hidden, device="cuda")
    assert lib.infer_moe_weighted_accumulate_slots_f32_batch_on_stream(idx.data_ptr(), wts.data_ptr(), down_t.data_ptr(), ones.data_ptr(),
                                                                       acc.data_ptr(), tokens, hidden, top_k, None) == 0
    torch.cuda.synchronize()
    # host evaluation
    oi, ow = oracle.moe_topk(logits, top_k, True)
    assert np.array_equal(idx.cpu().numpy().view(np.uint32), oi)
    ref_acc = np.zeros((tokens, hidden))
    for t in range(tokens):
        for slot in range(top_k):
            e = int(oi[t, slot])
            g_u = gu[e][3] @ x[t].astype(np.float64)
            got = gate_up[t * top_k + slot].cpu().numpy()
            ok, stats = gemm_close(got, g_u, rel=1e-4, abs_frac=1e-4)
            assert ok, stats
            g32 = got[:inter].astype(np.float64)
            a = g32 / (1 + np.exp(-g32)) * got[inter:].astype(np.float64)
            assert np.allclose(act[t * top_k + slot].cpu().numpy(), a, rtol=1e-5, atol=1e-7)
            d = dn[e][3] @ act[t * top_k + slot].cpu().numpy().astype(np.float64)
            ok, stats = gemm_close(down[t * top_k + slot].cpu().numpy(), d, rel=1e-4, abs_frac=1e-4)
            assert ok, stats
            ref_acc[t] += down[t * top_k + slot].cpu().numpy().astype(np.float64) * float(ow[t, slot])
    assert np.allclose(acc.cpu().numpy(), ref_acc, rtol=1e-5, atol=1e-6)
    fin = residual + ref_acc + shared_out * (1 / (1 + np.exp(-shared_logit.astype(np.float64))))[:, None]
    assert np.allclose(out.cpu().numpy(), fin, rtol=1e-2, atol=1e-2)  # bf16 precision by contract
    assert np.array_equal(out.cpu().numpy(), oracle.bf16_round(out.cpu().numpy()))
    # a slot whose expert is outside the table is skipped, and null arguments are rejected before any launch
    bad = torch.full((top_k,), experts + 3, dtype=torch.int32, device="cuda")
    before = gate_up[:top_k].clone()
    assert lib.infer_nvfp4_w4a16_grouped_matvec_f32_on_stream(bad.data_ptr(), xd[0].data_ptr(), gu_w.data_ptr(), gu_s.data_ptr(), gu_g.data_ptr(),
                                                              gate_up_t.data_ptr(), experts, top_k, 2 * inter, hidden, None) == 0
    torch.cuda.synchronize()
    assert torch.equal(gate_up[:top_k], before)
    assert lib.infer_nvfp4_w4a16_grouped_matvec_f32_on_stream(None, xd[0].data_ptr(), gu_w.data_ptr(), gu_s.data_ptr(), gu_g.data_ptr(),
                                                              gate_up_t.data_ptr(), experts, top_k, 2 * inter, hidden, None) == 1


def test_reuse_matvec_over_sorted_routes(lib, oracle):
    # crates/eider-cuda/src/ffi.rs:3333: routes sorted by expert; every route has its own input and output vector, found
    # through the tables by route id; equals the per-slot grouped-inputs GEMV on the same operands bit for bit
    import torch
    experts, routes, n, k = 6, 23, 200, 512
    rng = np.random.default_rng(5)
    ws = make_experts(oracle, rng, experts, n, k)
    w_dev = [(dev(p), dev(s)) for p, s, _, _ in ws]
    w_t, s_t = table([a for a, _ in w_dev]), table([b for _, b in w_dev])
    g_d = dev(np.array([g for _, _, g, _ in ws], np.float32))
    expert_of = rng.integers(0, experts, routes).astype(np.uint32)
    expert_of[expert_of == 2] = 3  # one expert receives nothing
    order = np.argsort(expert_of, kind="stable").astype(np.uint32)
    sorted_experts = expert_of[order]
    offsets = np.concatenate([[0], np.cumsum(np.bincount(expert_of, minlength=experts))]).astype(np.uint32)
    x = rng.standard_normal((routes, k)).astype(np.float32)
    xd = dev(x)
    y = torch.zeros(routes, n, device="cuda")
    x_t, y_t = table(list(xd)), table(list(y))
    i32 = lambda a: dev(np.ascontiguousarray(a, np.uint32).view(np.int32))
    sr, se, off = i32(order), i32(sorted_experts), i32(offsets)
    assert lib.infer_nvfp4_w4a16_reuse_matvec_f32_on_stream(sr.data_ptr(), se.data_ptr(), off.data_ptr(), x_t.data_ptr(), w_t.data_ptr(),
                                                            s_t.data_ptr(), g_d.data_ptr(), y_t.data_ptr(), routes, experts, n, k, None) == 0
    y2 = torch.zeros(routes, n, device="cuda")
    y2_t = table(list(y2))
    eo = i32(expert_of)
    assert lib.infer_nvfp4_w4a16_grouped_inputs_matvec_f32_on_stream(eo.data_ptr(), x_t.data_ptr(), w_t.data_ptr(), s_t.data_ptr(), g_d.data_ptr(),
                                                                     y2_t.data_ptr(), experts, routes, n, k, None) == 0
    torch.cuda.synchronize()
    assert torch.equal(y, y2)
    for r in range(routes):
        ok, stats = gemm_close(y[r].cpu().numpy(), ws[int(expert_of[r])][3] @ x[r].astype(np.float64), rel=1e-4, abs_frac=1e-4)
        assert ok, (r, stats)
    assert lib.infer_nvfp4_w4a16_reuse_matvec_f32_on_stream(sr.data_ptr(), se.data_ptr(), None, x_t.data_ptr(), w_t.data_ptr(), s_t.data_ptr(),
                                                            g_d.data_ptr(), y_t.data_ptr(), routes, experts, n, k, None) == 1
    # the single-token warp-rows form (ffi.rs:3296) is the batch form with one row
    p, s_, g, deq = ws[0]
    y1 = torch.zeros(n, device="cuda")
    assert lib.infer_nvfp4_w4a16_matvec_f32_warp_rows_on_stream(xd[0].data_ptr(), w_dev[0][0].data_ptr(), w_dev[0][1].data_ptr(), y1.data_ptr(),
                                                                n, k, g, 8, None) == 0
    torch.cuda.synchronize()
    ok, stats = gemm_close(y1.cpu().numpy(), deq @ x[0].astype(np.float64), rel=1e-4, abs_frac=1e-4)
    assert ok, stats


def test_fp8_moe_slots(lib, oracle):
    # crates/eider-cuda/src/ffi.rs:3163-3196: gate/up GEMV over a shared FP8 activation, SiLU * up -> per-slot dynamic FP8,
    # down GEMV over per-slot activations; against a host evaluation of the same codes (every product is exact)
    import torch
    experts, slots, hidden, inter = 5, 3, 528, 272
    rng = np.random.default_rng(23)

    def codes(shape):
        c = rng.integers(0, 256, shape).astype(np.uint8)
        c[(c & 0x7f) == 0x7f] = 0x31
        return c

    gate = [codes((inter, hidden)) for _ in range(experts)]
    up = [codes((inter, hidden)) for _ in range(experts)]
    down = [codes((hidden, inter)) for _ in range(experts)]
    gs = [(rng.random(inter) * 0.01 + 1e-3).astype(np.float32) for _ in range(experts)]
    us = [(rng.random(inter) * 0.01 + 1e-3).astype(np.float32) for _ in range(experts)]
    ds = [(rng.random(hidden) * 0.01 + 1e-3).astype(np.float32) for _ in range(experts)]
    x = codes(hidden)
    idx = np.array([4, 0, 2], np.uint32)
    dv = lambda arrs: [dev(a) for a in arrs]
    gate_d, up_d, down_d, gs_d, us_d, ds_d = dv(gate), dv(up), dv(down), dv(gs), dv(us), dv(ds)
    xd, xs = dev(x), dev(np.array([0.0625], np.float32))
    idx_d = dev(idx.view(np.int32))
    gu = torch.zeros(slots, 2 * inter, device="cuda")
    assert lib.infer_fp8_moe_grouped_gate_up_f32_on_stream(idx_d.data_ptr(), xd.data_ptr(), xs.data_ptr(), table(gate_d).data_ptr(),
                                                           table(gs_d).data_ptr(), table(up_d).data_ptr(), table(us_d).data_ptr(),
                                                           gu.data_ptr(), inter, hidden, slots, None) == 0
    q = torch.zeros(slots, inter, dtype=torch.uint8, device="cuda")
    qs = torch.zeros(slots, device="cuda")
    assert lib.infer_moe_silu_quantize_fp8_slots_f32_on_stream(gu.data_ptr(), q.data_ptr(), qs.data_ptr(), inter, slots, None) == 0
    out = torch.zeros(slots, hidden, device="cuda")
    assert lib.infer_fp8_moe_grouped_down_f32_on_stream(idx_d.data_ptr(), q.data_ptr(), qs.data_ptr(), table(down_d).data_ptr(),
                                                        table(ds_d).data_ptr(), table(list(out)).data_ptr(), hidden, inter, slots, None) == 0
    torch.cuda.synchronize()
    xv = oracle.e4m3_decode(x).astype(np.float64)
    for s_, e in enumerate(idx):
        g_ref = oracle.e4m3_decode(gate[e]).astype(np.float64) @ xv * 0.0625 * gs[e]
        u_ref = oracle.e4m3_decode(up[e]).astype(np.float64) @ xv * 0.0625 * us[e]
        got = gu[s_].cpu().numpy()
        ok, stats = gemm_close(got, np.concatenate([g_ref, u_ref]), rel=1e-4, abs_frac=1e-4)
        assert ok, stats
        # the quantizer on the device's own gate/up values: scale and codes follow the reference's formula
        g32, u32 = got[:inter], got[inter:]
        with np.errstate(over="ignore"):
            act = (g32 / (np.float32(1.0) + np.exp(-g32.astype(np.float32)))).astype(np.float32) * u32
        scale = np.float32(np.abs(act).max()) / np.float32(448.0)
        assert abs(float(qs[s_].item()) - float(scale)) <= 1e-6 * float(scale)
        deq = oracle.e4m3_decode(q[s_].cpu().numpy()).astype(np.float64) * float(qs[s_].item())
        assert np.all(np.abs(deq - act) <= 0.07 * np.abs(act) + 2e-3 * float(scale) * 448)
        d_ref = oracle.e4m3_decode(down[e]).astype(np.float64) @ oracle.e4m3_decode(q[s_].cpu().numpy()).astype(np.float64) * float(qs[s_].item()) * ds[e]
        ok, stats = gemm_close(out[s_].cpu().numpy(), d_ref, rel=1e-4, abs_frac=1e-4)
        assert ok, stats
    assert lib.infer_moe_silu_quantize_fp8_slots_f32_on_stream(None, q.data_ptr(), qs.data_ptr(), inter, slots, None) == 1
    assert lib.infer_fp8_moe_grouped_down_f32_on_stream(idx_d.data_ptr(), q.data_ptr(), qs.data_ptr(), table(down_d).data_ptr(),
                                                        table(ds_d).data_ptr(), table(list(out)).data_ptr(), hidden, inter + 8, slots, None) == 1


def test_decode_moe_w4a4_slots(lib, oracle):
    # the W4A4 decode variant: quantized activation row, indexed expert weights with tiled scales, per-expert alpha;
    # then SiLU * up -> NVFP4 with simple scales per slot, bit-exact against the host quantizer on the device's own values
    import torch

    from eider_b200 import ops
    experts, top_k, hidden, inter = 8, 4, 1024, 384
    rng = np.random.default_rng(7)
    gu = make_experts(oracle, rng, experts, 2 * inter, hidden)
    wds = [ops.ModelOptWeight.from_checkpoint(dev(p), dev(s), g) for p, s, g, _ in gu]
    w_t, s_t = table([w.packed for w in wds]), table([w.scales_tiled for w in wds])
    alpha = dev(np.array([g for _, _, g, _ in gu], np.float32))
    x = rng.standard_normal((1, hidden)).astype(np.float32)
    xp, xs = oracle.quantize_nvfp4(x, 1.0)
    xpd, xsd = dev(xp), dev(xs)
    idx = dev(np.array([5, 0, 7, 2], np.uint32).view(np.int32))
    gate_up = torch.zeros(top_k, 2 * inter, device="cuda")
    gate_up_t = table(list(gate_up))
    plan = lib.infer_cutlass_fp4_grouped_gemv_f32_create(2 * inter, hidden, top_k)
    assert plan and lib.infer_cutlass_fp4_grouped_gemv_f32_supported(2 * inter, hidden, top_k) == 1
    assert lib.infer_cutlass_fp4_grouped_gemv_f32_indexed_a_tiled_scales_on_stream(plan, idx.data_ptr(), w_t.data_ptr(), s_t.data_ptr(),
                                                                                   alpha.data_ptr(), experts, xpd.data_ptr(), xsd.data_ptr(),
                                                                                   None, gate_up_t.data_ptr(), None) == 0
    flat = torch.zeros(top_k, 2 * inter, device="cuda")
    first = table([w.packed for w in wds[:top_k]]), table([w.scales_tiled for w in wds[:top_k]])
    assert lib.infer_cutlass_fp4_grouped_gemv_f32_contiguous_b_on_stream(plan, first[0].data_ptr(), first[1].data_ptr(), xpd.data_ptr(),
                                                                         xsd.data_ptr(), flat.data_ptr(), 0.5, None) == 0
    torch.cuda.synchronize()
    xdq = oracle.dequantize_tiled(xp, xs)[0].astype(np.float64)
    for slot, e in enumerate([5, 0, 7, 2]):
        ok, stats = gemm_close(gate_up[slot].cpu().numpy(), gu[e][3] @ xdq, rel=1e-4, abs_frac=1e-4)
        assert ok, stats
    for g in range(top_k):
        ok, stats = gemm_close(flat[g].cpu().numpy(), gu[g][3] / gu[g][2] * 0.5 @ xdq, rel=1e-4, abs_frac=1e-4)
        assert ok, stats
    lib.infer_cutlass_fp4_grouped_gemv_f32_destroy(plan)
    # per-slot SiLU * up -> NVFP4, simple scales
    in_scales = dev(np.full(experts, 0.25, np.float32))
    ones = torch.ones(experts, device="cuda")
    packed = torch.zeros(top_k, inter // 2, dtype=torch.uint8, device="cuda")
    scales = torch.zeros(top_k, inter // 16, dtype=torch.uint8, device="cuda")
    act = torch.zeros(top_k, inter, device="cuda")
    assert lib.infer_moe_silu_slots_f32_on_stream(idx.data_ptr(), gate_up_t.data_ptr(), table(list(act)).data_ptr(), ones.data_ptr(), inter, top_k, None) == 0
    assert lib.infer_moe_silu_quantize_slots_nvfp4_simple_scales_on_stream(idx.data_ptr(), gate_up_t.data_ptr(), table(list(packed)).data_ptr(),
                                                                           table(list(scales)).data_ptr(), in_scales.data_ptr(), ones.data_ptr(),
                                                                           inter, top_k, None) == 0
    torch.cuda.synchronize()
    for slot in range(top_k):
        p_ref, s_ref = oracle.quantize_nvfp4_vector_simple_scales(act[slot].cpu().numpy(), 0.25)
        assert np.array_equal(packed[slot].cpu().numpy(), p_ref) and np.array_equal(scales[slot].cpu().numpy(), s_ref)


@pytest.mark.parametrize("n,k", [(1000, 512), (151936, 2048)])
def test_lm_head_top1(lib, oracle, n, k):
    # crates/eider-cuda/src/ffi.rs:3473: the arg-max equals the arg-max of the full GEMV (ties to the lower row)
    import torch

    from eider_b200 import ops
    g = torch.Generator(device="cuda").manual_seed(n)
    w = ops.ModelOptWeight.quantize(torch.randn(n, k, device="cuda", generator=g) * 0.02)
    x = torch.randn(1, k, device="cuda", generator=g)
    logits = ops.nvfp4_w4a16_matvec(x, w)  # the exact-f32 GEMV of the same library: same products, same sum order per row
    sv = torch.zeros(2048, device="cuda")
    si = torch.zeros(2048, dtype=torch.int32, device="cuda")
    out_i = torch.zeros(1, dtype=torch.int32, device="cuda")
    out_v = torch.zeros(1, device="cuda")
    for scratch_len in (2048, 7):
        assert lib.infer_nvfp4_w4a16_top1_f32_on_stream(x.data_ptr(), w.packed.data_ptr(), w.scales_row_major.data_ptr(), sv.data_ptr(),
                                                        si.data_ptr(), scratch_len, out_i.data_ptr(), out_v.data_ptr(), n, k, w.weight_scale_2,
                                                        8, None) == 0
        torch.cuda.synchronize()
        best = int(torch.argmax(logits[0]).item())
        assert int(out_i.item()) == best
        assert abs(float(out_v.item()) - float(logits[0, best].item())) <= 1e-5 * abs(float(logits[0, best].item())) + 1e-7
    # ties: two identical rows, the lower one wins
    w.packed[n - 1] = w.packed[best]
    w.scales_row_major[n - 1] = w.scales_row_major[best]
    assert lib.infer_nvfp4_w4a16_top1_f32_on_stream(x.data_ptr(), w.packed.data_ptr(), w.scales_row_major.data_ptr(), sv.data_ptr(), si.data_ptr(),
                                                    2048, out_i.data_ptr(), out_v.data_ptr(), n, k, w.weight_scale_2, 8, None) == 0
    torch.cuda.synchronize()
    assert int(out_i.item()) == min(best, n - 1)
    assert lib.infer_nvfp4_w4a16_top1_f32_on_stream(x.data_ptr(), w.packed.data_ptr(), w.scales_row_major.data_ptr(), sv.data_ptr(), si.data_ptr(),
                                                    2048, out_i.data_ptr(), out_v.data_ptr(), n, k, w.weight_scale_2, 5, None) == 1


def test_decode_moe_operator(lib, oracle):
    # the host mirror composes the same calls for one token
    import torch

    from eider_b200 import ops
    experts, top_k, hidden, inter = 8, 2, 256, 128
    rng = np.random.default_rng(2)
    gu = make_experts(oracle, rng, experts, 2 * inter, hidden)
    dn = make_experts(oracle, rng, experts, hidden, inter)
    layer = ops.DecodeMoe([ops.ModelOptWeight.from_checkpoint(dev(p), dev(s), g) for p, s, g, _ in gu],
                          [ops.ModelOptWeight.from_checkpoint(dev(p), dev(s), g) for p, s, g, _ in dn], top_k)
    x, logits = rng.standard_normal(hidden).astype(np.float32), rng.standard_normal(experts).astype(np.float32)
    shared, res = rng.standard_normal(hidden).astype(np.float32), rng.standard_normal(hidden).astype(np.float32)
    gate = np.array([0.3], np.float32)
    out = layer.run(dev(x), dev(logits), dev(gate), dev(shared), dev(res)).cpu().numpy()
    idx, w = oracle.moe_topk(logits[None], top_k, True)
    routed = np.zeros(hidden)
    for slot in range(top_k):
        e = int(idx[0, slot])
        g_u = gu[e][3] @ x.astype(np.float64)
        a = g_u[:inter] / (1 + np.exp(-g_u[:inter])) * g_u[inter:]
        routed += (dn[e][3] @ a) * float(w[0, slot])
    ref = res + routed + shared / (1 + np.exp(-0.3))
    assert np.allclose(out, ref, rtol=1e-2, atol=1e-2)
    assert np.array_equal(out, oracle.bf16_round(out))
