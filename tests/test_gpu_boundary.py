"""Entry points that keep the reference's names and argument lists (crates/eider-cuda/src/ffi.rs), called through ctypes
exactly as a binding would call them, against the CPU oracle: the scratch-free route sort, the direct sorted-row
quantizers (plain, calibrated, ReLU^2, GELU), the RMSNorm gather, the pointer tables, the plan-less W4A4 GEMV and the
plan-less FP8 linears."""
import ctypes

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


def i32(a):
    return dev(np.ascontiguousarray(a, np.uint32).view(np.int32))


def u32(t):
    return t.cpu().numpy().view(np.uint32)


def deq_dot(matrix, vector):
    return matrix @ vector


def sort_on_device(lib, ind, experts):
    import torch
    routes = ind.size
    z = lambda n: torch.zeros(n, dtype=torch.int32, device="cuda")
    out = dict(counts=z(experts), offsets=z(experts + 1), cursors=z(experts), sorted_routes=z(routes), sorted_experts=z(routes),
               inverse=z(routes))
    ind_d = i32(ind)
    st = lib.infer_moe_sort_routes_on_stream(ind_d.data_ptr(), out["counts"].data_ptr(), out["offsets"].data_ptr(),
                                             out["cursors"].data_ptr(), out["sorted_routes"].data_ptr(),
                                             out["sorted_experts"].data_ptr(), out["inverse"].data_ptr(), routes, experts, None)
    assert st == 0
    torch.cuda.synchronize()
    return out


def moe_buffers(routes, experts, k):
    import torch
    tile = 128 * ((k // 16 + 3) // 4 * 4)
    return (torch.zeros(routes, k // 2, dtype=torch.uint8, device="cuda"),
            torch.zeros(((routes + 127) // 128 + experts) * tile, dtype=torch.uint8, device="cuda"), tile)


@pytest.mark.parametrize("routes,experts", [(8, 4), (21, 5), (32768, 128), (65536, 1024)])
def test_reference_sort_call_matches_oracle(lib, oracle, routes, experts):
    # crates/eider-cuda/src/ffi.rs:1701; (65536, 1024) is exactly the 262144-entry limit of the built-in table
    rng = np.random.default_rng(routes)
    ind = (np.array([3, 1, 3, 0, 1, 2, 3, 2], np.uint32) if routes == 8 else rng.integers(0, experts, routes).astype(np.uint32))
    got = sort_on_device(lib, ind, experts)
    counts, offsets, sorted_routes, sorted_experts, inverse = oracle.moe_sort_routes(ind, experts)
    assert np.array_equal(u32(got["counts"]), counts)
    assert np.array_equal(u32(got["offsets"]), offsets)
    assert np.array_equal(u32(got["cursors"]), offsets[1:])  # where the reference's atomic cursors end up
    assert np.array_equal(u32(got["sorted_routes"]), sorted_routes)
    assert np.array_equal(u32(got["sorted_experts"]), sorted_experts)
    assert np.array_equal(u32(got["inverse"]), inverse)
    if routes == 8:
        assert counts.tolist() == [1, 2, 2, 3] and offsets.tolist() == [0, 1, 3, 5, 8]


def test_reference_sort_call_rejects_what_the_table_cannot_hold(lib):
    import torch
    routes, experts = 65536 + 256, 1024
    z = torch.zeros(routes + experts + 1, dtype=torch.int32, device="cuda")
    assert lib.infer_moe_sort_routes_on_stream(z.data_ptr(), z.data_ptr(), z.data_ptr(), z.data_ptr(), z.data_ptr(), z.data_ptr(),
                                               z.data_ptr(), routes, experts, None) == 1
    assert lib.infer_moe_sort_routes_on_stream(None, z.data_ptr(), z.data_ptr(), z.data_ptr(), z.data_ptr(), z.data_ptr(),
                                               z.data_ptr(), 8, 4, None) == 1


@pytest.mark.parametrize("gather", [1, 0])
@pytest.mark.parametrize("tokens,top,experts,k", [(7, 3, 5, 80), (512, 8, 16, 2048)])
def test_quantize_sorted_routes_matches_oracle(lib, oracle, tokens, top, experts, k, gather):
    # crates/eider-cuda/src/ffi.rs:1728: rows gathered by route, or already in sorted order
    import torch
    rng = np.random.default_rng(tokens + k)
    routes = tokens * top
    ind = rng.integers(0, experts, routes).astype(np.uint32)
    s = sort_on_device(lib, ind, experts)
    x = rng.standard_normal((tokens if gather else routes, k)).astype(np.float32)
    packed, scales, tile = moe_buffers(routes, experts, k)
    xd = dev(x)  # (device operands are held in names: a temporary's memory may be handed out again before the launch)
    st = lib.infer_moe_quantize_sorted_routes_nvfp4_on_stream(xd.data_ptr(), s["sorted_routes"].data_ptr(), s["sorted_experts"].data_ptr(),
                                                              s["offsets"].data_ptr(), packed.data_ptr(), scales.data_ptr(), routes, top, k,
                                                              tile, gather, None)
    assert st == 0
    torch.cuda.synchronize()
    _, offsets, sorted_routes, sorted_experts, _ = oracle.moe_sort_routes(ind, experts)
    p_ref, s_ref = oracle.moe_gather_quantize(x, sorted_routes, sorted_experts, offsets, top, experts, gather_rows=bool(gather))
    assert np.array_equal(packed.cpu().numpy(), p_ref)
    assert np.array_equal(scales.cpu().numpy(), s_ref)


@pytest.mark.parametrize("relu", [0, 1])
def test_calibrated_quantize_reference_fixture(lib, oracle, relu):
    # crates/eider-cuda/src/kernels/non_gemm.rs:15168-15249: 7 tokens x top-3 x 5 experts x K = 80, index pattern
    # [0, 4, 1, 0, 1, 4, 3], per-expert scales [.125, .25, 1, 2, .5]
    import torch
    rows, top, experts, k = 7, 3, 5, 80
    routes = rows * top
    ind = np.array([[0, 4, 1, 0, 1, 4, 3][i % 7] for i in range(routes)], np.uint32)
    scales_in = np.array([0.125, 0.25, 1.0, 2.0, 0.5], np.float32)
    values = ((np.arange(rows * k) % 29).astype(np.float32) / 16.0 - 0.75).astype(np.float32).reshape(rows, k)
    sorted_bf16 = oracle.bf16_round(((np.arange(routes * k) % 37).astype(np.float32) / 16.0 - 1.0).astype(np.float32)).reshape(routes, k)
    s = sort_on_device(lib, ind, experts)
    packed, scales, tile = moe_buffers(routes, experts, k)
    src = dev(sorted_bf16, torch.bfloat16) if relu else dev(values)
    scales_d = dev(scales_in)
    st = lib.infer_moe_calibrated_quantize_on_stream(src.data_ptr(), scales_d.data_ptr(), s["sorted_routes"].data_ptr(),
                                                     s["sorted_experts"].data_ptr(), s["offsets"].data_ptr(), packed.data_ptr(),
                                                     scales.data_ptr(), routes, top, k, tile, relu, None)
    assert st == 0
    torch.cuda.synchronize()
    _, offsets, sorted_routes, sorted_experts, _ = oracle.moe_sort_routes(ind, experts)
    vals = oracle.moe_calibrated_values(sorted_bf16 if relu else values, scales_in, sorted_routes, sorted_experts, top, bool(relu))
    p_ref, s_ref = oracle.moe_quantize_rows_into_expert_tiles(vals, sorted_experts, offsets, experts)
    assert np.array_equal(packed.cpu().numpy(), p_ref)
    assert np.array_equal(scales.cpu().numpy(), s_ref)
    # and the reference's own per-row statement: each sorted row equals the host quantizer on value / scale
    for srt in range(routes):
        e = int(sorted_experts[srt])
        row = (np.maximum(sorted_bf16[srt], 0) ** 2 if relu else values[int(sorted_routes[srt]) // top]) / scales_in[e]
        pr, _ = oracle.quantize_nvfp4(row[None].astype(np.float32), 1.0)
        assert np.array_equal(packed.cpu().numpy()[srt], pr[0])


def test_gelu_sorted_routes_matches_staged_quantizer(lib, oracle):
    # crates/eider-cuda/src/ffi.rs:1742: GELU-tanh(gate) * up of sorted bf16 rows == the same values through the f32 operator
    # and the direct sorted-row quantizer (byte for byte), and the CPU oracle up to tanh's last place
    import torch
    routes, experts, k = 600, 9, 768
    rng = np.random.default_rng(3)
    ind = rng.integers(0, experts, routes).astype(np.uint32)
    s = sort_on_device(lib, ind, experts)
    gate = oracle.bf16_round((rng.standard_normal((routes, k)) * 2).astype(np.float32))
    up = oracle.bf16_round(rng.standard_normal((routes, k)).astype(np.float32))
    fused_p, fused_s, tile = moe_buffers(routes, experts, k)
    gate_bf, up_bf, gate_f, up_f = dev(gate, torch.bfloat16), dev(up, torch.bfloat16), dev(gate), dev(up)
    st = lib.infer_moe_gelu_tanh_mul_quantize_sorted_routes_nvfp4_on_stream(
        gate_bf.data_ptr(), up_bf.data_ptr(), s["sorted_experts"].data_ptr(), s["offsets"].data_ptr(),
        fused_p.data_ptr(), fused_s.data_ptr(), routes, k, tile, None)
    assert st == 0
    act = torch.empty(routes, k, device="cuda")
    assert lib.infer_gelu_tanh_mul_f32_on_stream(gate_f.data_ptr(), up_f.data_ptr(), act.data_ptr(), routes * k, None) == 0
    staged_p, staged_s, _ = moe_buffers(routes, experts, k)
    assert lib.infer_moe_quantize_sorted_routes_nvfp4_on_stream(act.data_ptr(), s["sorted_routes"].data_ptr(), s["sorted_experts"].data_ptr(),
                                                                s["offsets"].data_ptr(), staged_p.data_ptr(), staged_s.data_ptr(), routes, 1, k,
                                                                tile, 0, None) == 0
    torch.cuda.synchronize()
    assert torch.equal(fused_p, staged_p) and torch.equal(fused_s, staged_s)
    _, offsets, _, sorted_experts, _ = oracle.moe_sort_routes(ind, experts)
    p_ref, _ = oracle.moe_quantize_rows_into_expert_tiles(oracle.gelu_tanh_mul(gate, up), sorted_experts, offsets, experts)
    assert np.count_nonzero(fused_p.cpu().numpy() != p_ref) / p_ref.size < 2e-3


def test_gather_rms_norm_quantize_equals_norm_then_gather(lib, oracle):
    # crates/eider-cuda/src/ffi.rs:1765 == RMSNorm -> NVFP4 of every token (unit scale), then the byte scatter
    import torch
    tokens, top, experts, k = 96, 4, 8, 1024
    routes = tokens * top
    rng = np.random.default_rng(5)
    ind = rng.integers(0, experts, routes).astype(np.uint32)
    s = sort_on_device(lib, ind, experts)
    x = rng.standard_normal((tokens, k)).astype(np.float32)
    w = rng.uniform(0.5, 1.5, k).astype(np.float32)
    xd, wd = dev(x), dev(w)
    src_p = torch.zeros(tokens, k // 2, dtype=torch.uint8, device="cuda")
    from eider_b200 import ops
    src_s = torch.zeros(ops.scale_layout_len(tokens, k), dtype=torch.uint8, device="cuda")
    packed, scales, tile = moe_buffers(routes, experts, k)
    st = lib.infer_moe_gather_rms_norm_quantize_sorted_routes_nvfp4_on_stream(
        xd.data_ptr(), wd.data_ptr(), s["sorted_routes"].data_ptr(), s["sorted_experts"].data_ptr(), s["offsets"].data_ptr(),
        src_p.data_ptr(), src_s.data_ptr(), packed.data_ptr(), scales.data_ptr(), tokens, routes, top, k, tile, 1e-6, None)
    assert st == 0
    # staged on the device: norm to f32, then the direct gather quantizer
    normed = torch.empty_like(xd)
    assert lib.infer_rms_norm_f32_on_stream(xd.data_ptr(), wd.data_ptr(), normed.data_ptr(), tokens, k, 1e-6, None) == 0
    p2, s2, _ = moe_buffers(routes, experts, k)
    assert lib.infer_moe_quantize_sorted_routes_nvfp4_on_stream(normed.data_ptr(), s["sorted_routes"].data_ptr(), s["sorted_experts"].data_ptr(),
                                                                s["offsets"].data_ptr(), p2.data_ptr(), s2.data_ptr(), routes, top, k, tile, 1,
                                                                None) == 0
    torch.cuda.synchronize()
    assert torch.equal(packed, p2) and torch.equal(scales, s2)


def test_grouped_pointer_tables(lib):
    # crates/eider-cuda/src/ffi.rs:1799 (kernel non_gemm.cu:3066-3083): table[e] = base + offset of expert e
    import torch
    experts, k, n = 6, 256, 384
    tile = 128 * ((k // 16 + 3) // 4 * 4)
    offsets = np.array([0, 5, 5, 140, 141, 300, 301], np.uint32)
    routes = int(offsets[-1])
    packed = torch.zeros(routes, k // 2, dtype=torch.uint8, device="cuda")
    scales = torch.zeros(((routes + 127) // 128 + experts) * tile, dtype=torch.uint8, device="cuda")
    out = torch.zeros(routes, n, dtype=torch.bfloat16, device="cuda")
    tables = [torch.zeros(experts, dtype=torch.int64, device="cuda") for _ in range(3)]
    st = lib.infer_moe_grouped_pointer_tables_on_stream(i32(offsets).data_ptr(), packed.data_ptr(), scales.data_ptr(), out.data_ptr(),
                                                        tables[0].data_ptr(), tables[1].data_ptr(), tables[2].data_ptr(), experts, k, n,
                                                        tile, None)
    assert st == 0
    torch.cuda.synchronize()
    for e in range(experts):
        off = int(offsets[e])
        assert int(tables[0][e]) == packed.data_ptr() + off * (k // 2)
        assert int(tables[1][e]) == scales.data_ptr() + ((off + 127) // 128 + e) * tile
        assert int(tables[2][e]) == out.data_ptr() + off * n * 2
    assert lib.infer_moe_grouped_pointer_tables_on_stream(None, packed.data_ptr(), scales.data_ptr(), out.data_ptr(), tables[0].data_ptr(),
                                                          tables[1].data_ptr(), tables[2].data_ptr(), experts, k, n, tile, None) == 1


@pytest.mark.parametrize("tokens,experts,top_k,hidden,out_features", [(64, 6, 2, 256, 384), (300, 16, 4, 512, 256), (1024, 32, 8, 2048, 1536)])
def test_reference_grouped_gemm_over_pointer_tables(lib, oracle, tokens, experts, top_k, hidden, out_features):
    # crates/eider-cuda/src/ffi.rs:643-667 (CutlassFp4GroupedGemmPlan::run_on_stream, cublaslt/fp4_tn.rs:1218-1262): seven
    # device arrays of per-expert pointers and counts.  The row / scale / output tables come from the reference's own
    # table kernel, the weight tables from the stacked checkpoint tensors; the result must equal the base-pointer form of
    # the same GEMM bit for bit, and sampled experts are checked against the host product.
    import torch
    from eider_b200 import ops
    g = torch.Generator(device="cuda").manual_seed(tokens + experts)
    x = torch.randn(tokens, hidden, device="cuda", generator=g)
    logits = torch.randn(tokens, experts, device="cuda", generator=g)
    logits[:, 1] = -50.0  # an expert that receives nothing
    w = ops.GroupedNvfp4Weights.quantize(torch.randn(experts, out_features, hidden, device="cuda", generator=g) * 0.02)
    idx, _ = ops.moe_topk(logits, top_k, True)
    routes = ops.MoeSortedRoutes(tokens * top_k, experts)
    routes.sort(idx.reshape(-1))
    rows = ops.MoeSortedNvfp4Rows(tokens * top_k, experts, hidden, tokens)
    rows.gather_quantize(x, routes, top_k)
    plan = ops.Fp4GroupedGemmPlan(out_features, tokens * top_k, hidden, experts)
    want = plan.run(rows, w, routes)
    torch.cuda.synchronize()

    n_routes = tokens * top_k
    got = torch.full((n_routes, out_features), 7.0, dtype=torch.bfloat16, device="cuda")
    z = lambda: torch.zeros(experts, dtype=torch.int64, device="cuda")
    a_tbl, as_tbl, out_tbl = z(), z(), z()
    assert lib.infer_moe_grouped_pointer_tables_on_stream(routes.expert_offsets.data_ptr(), rows.packed.data_ptr(), rows.scales.data_ptr(),
                                                          got.data_ptr(), a_tbl.data_ptr(), as_tbl.data_ptr(), out_tbl.data_ptr(), experts,
                                                          hidden, out_features, rows.tile_bytes, None) == 0
    sf_per_expert = (out_features // 128) * 128 * ((hidden // 16 + 3) // 4 * 4)
    e_ids = torch.arange(experts, device="cuda", dtype=torch.int64)
    b_tbl = w.packed.data_ptr() + e_ids * (out_features * hidden // 2)
    bs_tbl = w.scales_tiled.data_ptr() + e_ids * sf_per_expert
    alpha_tbl = w.alpha.data_ptr() + e_ids * 4
    counts = routes.expert_counts
    assert lib.infer_cutlass_fp4_grouped_gemm_supported(out_features, n_routes, hidden, experts) == 1
    tplan = lib.infer_cutlass_fp4_grouped_gemm_create(out_features, n_routes, hidden, experts)
    assert tplan
    try:
        for _ in range(2):  # the per-group maps are rewritten by every call
            st = lib.infer_cutlass_fp4_grouped_gemm_on_stream(tplan, a_tbl.data_ptr(), as_tbl.data_ptr(), b_tbl.data_ptr(), bs_tbl.data_ptr(),
                                                              out_tbl.data_ptr(), alpha_tbl.data_ptr(), counts.data_ptr(), None)
            assert st == 0
        torch.cuda.synchronize()
        status = ctypes.c_uint32(1)
        assert lib.eider_b200_grouped_plan_status(tplan, ctypes.byref(status)) == 0 and status.value == 0
        assert torch.equal(got, want)
        # nothing is read back to the host and nothing is allocated: the call records into a CUDA graph and replays
        got.fill_(3.0)
        side = torch.cuda.Stream()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            with torch.cuda.graph(graph, stream=side):
                assert lib.infer_cutlass_fp4_grouped_gemm_on_stream(tplan, a_tbl.data_ptr(), as_tbl.data_ptr(), b_tbl.data_ptr(),
                                                                    bs_tbl.data_ptr(), out_tbl.data_ptr(), alpha_tbl.data_ptr(),
                                                                    counts.data_ptr(), side.cuda_stream) == 0
            graph.replay()
        torch.cuda.synchronize()
    finally:
        lib.infer_cutlass_fp4_grouped_gemm_destroy(tplan)
    assert torch.equal(got, want)
    assert lib.infer_cutlass_fp4_grouped_gemm_on_stream(None, a_tbl.data_ptr(), as_tbl.data_ptr(), b_tbl.data_ptr(), bs_tbl.data_ptr(),
                                                        out_tbl.data_ptr(), alpha_tbl.data_ptr(), counts.data_ptr(), None) == 1


@pytest.mark.parametrize("m,k", [(13824, 5120), (5120, 13824), (300, 96)])
def test_reference_w4a4_gemv_f32(lib, oracle, m, k):
    # crates/eider-cuda/src/ffi.rs:576-588 (test crates/eider-cuda/src/cublaslt/fp4_tn.rs:1652-1712): both operands NVFP4,
    # f32 output; the oracle is the host dequantize + f32 dot product
    import torch

    from eider_b200 import ops
    rng = np.random.default_rng(m + k)
    w = (rng.standard_normal((m, k)) * 0.02).astype(np.float32)
    wp, ws, g = oracle.quantize_weight(w)
    x = rng.standard_normal((1, k)).astype(np.float32)
    xp, xs = oracle.quantize_nvfp4(x, 1.0)
    wd = ops.ModelOptWeight.from_checkpoint(dev(wp), dev(ws), float(g))
    c = torch.zeros(m, device="cuda")
    d = torch.full((m + 8,), -77.0, device="cuda")
    xpd, xsd = dev(xp), dev(xs)
    assert lib.infer_cutlass_fp4_gemv_f32_supported(m, k) == 1
    st = lib.infer_cutlass_fp4_gemv_f32_on_stream(wd.packed.data_ptr(), wd.scales_tiled.data_ptr(), xpd.data_ptr(), xsd.data_ptr(),
                                                  c.data_ptr(), d.data_ptr(), m, k, float(g), None)
    assert st == 0
    torch.cuda.synchronize()
    ref = oracle.matmul_nt(oracle.dequantize_tiled(xp, xs), oracle.dequantize_weight(wp, ws), alpha=float(g))[0]
    ok, stats = gemm_close(d[:m].cpu().numpy(), ref, rel=1e-3, abs_frac=1e-3)  # every product is exact; only the accumulation differs
    assert ok, stats
    assert torch.all(d[m:] == -77.0)  # guard elements behind the output stay untouched
    assert lib.infer_cutlass_fp4_gemv_f32_supported(m, k + 16) == 0
    assert lib.infer_cutlass_fp4_gemv_f32_on_stream(wd.packed.data_ptr(), wd.scales_tiled.data_ptr(), xpd.data_ptr(), xsd.data_ptr(),
                                                    None, d.data_ptr(), m, k, float(g), None) == 1


def test_reference_fp8_linear_shims(lib, oracle):
    # crates/eider-cuda/src/ffi.rs:3131, :3151, :3239 at the QKV shape of the decode config
    import torch
    n, k = 7168, 5120
    rng = np.random.default_rng(11)
    w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    wq, sw = oracle.quantize_fp8_weight(w)
    x = rng.standard_normal((1, k)).astype(np.float32)
    xq, sx = oracle.quantize_fp8_dynamic(x)
    ref = oracle.fp8_linear(xq, sx, wq, sw)[0]
    wd, swd, xd = dev(wq), dev(sw), dev(x)
    y = torch.zeros(n, device="cuda")
    assert lib.infer_fp8_linear_channel_scaled_dynamic_f32_on_stream(xd.data_ptr(), wd.data_ptr(), swd.data_ptr(), y.data_ptr(), n, k, None) == 0
    torch.cuda.synchronize()
    ok, stats = gemm_close(y.cpu().numpy(), ref, rel=1e-3, abs_frac=1e-3)
    assert ok, stats
    y2 = torch.zeros(n, device="cuda")
    q_out = torch.zeros(k, dtype=torch.uint8, device="cuda")
    s_out = torch.zeros(1, device="cuda")
    assert lib.infer_fp8_linear_channel_scaled_dynamic_quantized_f32_configured_on_stream(
        xd.data_ptr(), q_out.data_ptr(), wd.data_ptr(), swd.data_ptr(), s_out.data_ptr(), y2.data_ptr(), n, k, 256, None) == 0
    torch.cuda.synchronize()
    assert np.array_equal(q_out.cpu().numpy(), xq[0]) and float(s_out.item()) == float(sx[0])
    ok, stats = gemm_close(y2.cpu().numpy(), ref, rel=1e-3, abs_frac=1e-3)
    assert ok, stats
    # static activation scale, per-tensor weight scale
    xs = oracle.quantize_fp8_static(x, 0.03125)
    ref3 = oracle.fp8_linear(xs, np.array([0.03125], np.float32), wq, np.full(n, 0.5, np.float32))[0]
    y3 = torch.zeros(n, device="cuda")
    assert lib.infer_fp8_linear_w8a8_f32_on_stream(xd.data_ptr(), wd.data_ptr(), y3.data_ptr(), n, k, 0.5, 0.03125, None) == 0
    torch.cuda.synchronize()
    ok, stats = gemm_close(y3.cpu().numpy(), ref3, rel=1e-3, abs_frac=1e-3)
    assert ok, stats
    assert lib.infer_fp8_linear_w8a8_f32_on_stream(xd.data_ptr(), wd.data_ptr(), y3.data_ptr(), n, k, 0.5, 0.0, None) == 1


def test_reference_fp8_weight_only_linears(lib, oracle):
    # crates/eider-cuda/src/ffi.rs:3056-3147: f32 activations times E4M3 weights, scalar or per-row weight scale, single /
    # batch / pair / triple forms, and the "precomputed dynamic" form that quantizes the activation per tensor first
    import torch
    n, n2, n3, k, batch = 1000, 264, 72, 2064, 5
    rng = np.random.default_rng(17)
    ws = [rng.integers(0, 256, (r, k)).astype(np.uint8) for r in (n, n2, n3)]
    for w in ws:
        w[(w & 0x7f) == 0x7f] = 0x30  # no NaN codes
    deq = [oracle.e4m3_decode(w).astype(np.float64) for w in ws]
    x = rng.standard_normal((batch, k)).astype(np.float32)
    ch = (rng.random(n) * 0.01 + 0.001).astype(np.float32)
    wd = [dev(w) for w in ws]
    xd, chd = dev(x), dev(ch)
    y = torch.full((batch, n), -5.0, device="cuda")
    assert lib.infer_fp8_linear_f32_batch_on_stream(xd.data_ptr(), wd[0].data_ptr(), y.data_ptr(), batch, n, k, 0.25, 256, None) == 0
    y1 = torch.zeros(n, device="cuda")
    assert lib.infer_fp8_linear_f32_configured_on_stream(xd.data_ptr(), wd[0].data_ptr(), y1.data_ptr(), n, k, 0.25, 128, None) == 0
    yc = torch.zeros(batch, n, device="cuda")
    assert lib.infer_fp8_linear_channel_scaled_f32_batch_configured_on_stream(xd.data_ptr(), wd[0].data_ptr(), chd.data_ptr(), yc.data_ptr(),
                                                                              batch, n, k, 256, None) == 0
    yc1 = torch.zeros(n, device="cuda")
    assert lib.infer_fp8_linear_channel_scaled_f32_configured_on_stream(xd.data_ptr(), wd[0].data_ptr(), chd.data_ptr(), yc1.data_ptr(), n, k,
                                                                        256, None) == 0
    o = [torch.zeros(r, device="cuda") for r in (n, n2, n3)]
    assert lib.infer_fp8_linear_triple_f32_configured_on_stream(xd.data_ptr(), wd[0].data_ptr(), wd[1].data_ptr(), wd[2].data_ptr(),
                                                                o[0].data_ptr(), o[1].data_ptr(), o[2].data_ptr(), n, n2, n3, k, 0.25, 0.5,
                                                                2.0, 256, None) == 0
    p = [torch.zeros(r, device="cuda") for r in (n, n2)]
    assert lib.infer_fp8_linear_pair_f32_configured_on_stream(xd.data_ptr(), wd[0].data_ptr(), wd[1].data_ptr(), p[0].data_ptr(), p[1].data_ptr(),
                                                              n, n2, k, 0.25, 0.5, 256, None) == 0
    torch.cuda.synchronize()
    xr = x.astype(np.float64)
    for got, ref in ((y.cpu().numpy(), xr @ deq[0].T * 0.25), (yc.cpu().numpy(), xr @ deq[0].T * ch[None, :].astype(np.float64))):
        ok, stats = gemm_close(got, ref, rel=1e-4, abs_frac=1e-4)
        assert ok, stats
    assert torch.equal(y1, y[0]) and torch.equal(yc1, yc[0])
    for got, d, sc in ((o[0], deq[0], 0.25), (o[1], deq[1], 0.5), (o[2], deq[2], 2.0)):
        ok, stats = gemm_close(got.cpu().numpy(), deq_dot(d, xr[0]) * sc, rel=1e-4, abs_frac=1e-4)
        assert ok, stats
    assert torch.equal(p[0], o[0]) and torch.equal(p[1], o[1])
    # precomputed dynamic: input_scale[0] = amax / 448, then e4m3(x / scale) times the weights, times scale and the row scale
    xq, sx = oracle.quantize_fp8_dynamic(x[:1])
    s_out = torch.zeros(1, device="cuda")
    yd = torch.zeros(n, device="cuda")
    assert lib.infer_fp8_linear_channel_scaled_precomputed_dynamic_f32_on_stream(xd.data_ptr(), wd[0].data_ptr(), chd.data_ptr(),
                                                                                 s_out.data_ptr(), yd.data_ptr(), n, k, None) == 0
    torch.cuda.synchronize()
    assert float(s_out.item()) == float(sx[0])
    ref = (deq[0] @ oracle.e4m3_decode(xq[0]).astype(np.float64)) * float(sx[0]) * ch.astype(np.float64)
    ok, stats = gemm_close(yd.cpu().numpy(), ref, rel=1e-4, abs_frac=1e-4)
    assert ok, stats
    # rejected before any launch: null pointers, a thread count outside the reference's range, a row length off the 16 grid
    assert lib.infer_fp8_linear_f32_batch_on_stream(None, wd[0].data_ptr(), y.data_ptr(), batch, n, k, 0.25, 256, None) == 1
    assert lib.infer_fp8_linear_f32_batch_on_stream(xd.data_ptr(), wd[0].data_ptr(), y.data_ptr(), batch, n, k, 0.25, 48, None) == 1
    assert lib.infer_fp8_linear_f32_batch_on_stream(xd.data_ptr(), wd[0].data_ptr(), y.data_ptr(), batch, n, k - 8, 0.25, 256, None) == 1
    assert lib.infer_fp8_linear_channel_scaled_f32_configured_on_stream(xd.data_ptr(), wd[0].data_ptr(), None, yc1.data_ptr(), n, k, 256,
                                                                        None) == 1


@pytest.mark.parametrize("batch", [1, 7])
def test_block_scaled_fp8_linears(lib, oracle, batch):
    # crates/eider-cuda/native/deepseek4.cu:86-170: f32 activations x E4M3 weights x one scale per 128 x 128 block
    import torch
    n, k = 512, 1024
    rng = np.random.default_rng(batch)
    codes = rng.integers(0, 256, (n, k)).astype(np.uint8)
    codes[(codes & 0x7F) == 0x7F] = 0x30
    e8 = rng.integers(118, 131, (n // 128, k // 128)).astype(np.uint8)
    f32s = rng.uniform(0.01, 2.0, (n // 128, k // 128)).astype(np.float32)
    x = rng.standard_normal((batch, k)).astype(np.float32)
    wv = oracle.e4m3_decode(codes).astype(np.float64)
    xd, wd = dev(x), dev(codes)
    for name, scales, dense in (("infer_deepseek4_block_fp8_linear_f32_on_stream", e8,
                                 np.array([[oracle.e8m0_value(int(c)) for c in r] for r in e8], np.float64)),
                                ("infer_block_fp8_f32_scale_linear_f32_on_stream", f32s, f32s.astype(np.float64))):
        y = torch.full((batch, n + 4), -77.0, device="cuda")[:, :n].contiguous()
        sd = dev(scales)
        assert getattr(lib, name)(xd.data_ptr(), wd.data_ptr(), sd.data_ptr(), y.data_ptr(), batch, n, k, None) == 0
        torch.cuda.synchronize()
        ref = x.astype(np.float64) @ (wv * np.kron(dense, np.ones((128, 128)))).T
        ok, stats = gemm_close(y.cpu().numpy(), ref, rel=1e-4, abs_frac=1e-4)
        assert ok, (name, stats)
        assert getattr(lib, name)(xd.data_ptr(), wd.data_ptr(), sd.data_ptr(), y.data_ptr(), batch, n + 64, k, None) == 1
