"""Pins the CPU oracle to the reference's own known-answer vectors.

Each case names the reference test it restates (file:line inside the reference tree).
"""
import math
import struct

import numpy as np


def _f(bits):
    return struct.unpack("<f", struct.pack("<I", bits))[0]


# crates/eider-cuda/src/format.rs:395-445
E2M1_VALUES = [
    -math.inf, -99.0, -6.1, -6.0, -5.0, -3.5, -2.5, -1.75, -1.25, -0.75, -0.26, -0.25, -0.24, -0.0,
    0.0, 0.24, 0.25, 0.26, 0.75, 1.25, 1.26, 1.75, 2.5, 3.5, 5.0, 6.0, 6.1, 99.0, math.inf, math.nan,
]
for _b in [0x00000001, 0x007FFFFF, 0x00800000, 0x3E7FFFFF, 0x3E800000, 0x3EFFFFFF, 0x3F000000,
           0x3F7FFFFF, 0x3F800000, 0x40BFFFFF, 0x40C00000]:
    E2M1_VALUES += [_f(_b), -_f(_b)]


def test_pack_low_nibble_first(oracle):
    # format.rs:454-457
    assert oracle.pack_e2m1([1.0, -1.0]).tolist() == [0xA2]
    assert oracle.pack_e2m1([1.0, 0.0, -1.0]).tolist() == [0x02, 0x0A]


def test_e8m0(oracle):
    # format.rs:461-466
    assert oracle.e8m0_value(126) == 0.5
    assert oracle.e8m0_value(127) == 1.0
    assert oracle.e8m0_value(128) == 2.0
    assert math.isnan(oracle.e8m0_value(255))


def test_e2m1_tie_points(oracle):
    # ties go to the even code: 0.25->0, 0.75->1.0, 1.25->1.0, 1.75->2.0, 2.5->2.0, 3.5->4.0, 5.0->4.0
    expect = {0.25: 0, 0.75: 2, 1.25: 2, 1.75: 4, 2.5: 4, 3.5: 6, 5.0: 6, 6.1: 7, -0.25: 8}
    for v, c in expect.items():
        assert oracle.e2m1_code(v) == c, v
    assert oracle.e2m1_code(math.nan) == 7
    assert oracle.e2m1_code(-0.0) == 8


def test_ue4m3_known_codes(oracle):
    assert oracle.ue4m3_code(1.0) == 0x38
    assert oracle.ue4m3_code(448.0) == 0x7E
    assert oracle.ue4m3_code(1000.0) == 0x7E
    assert oracle.ue4m3_code(1e-4) == 0x00
    assert oracle.ue4m3_code(1e-3) == 0x01
    assert oracle.ue4m3_code(0.0) == 0
    assert oracle.ue4m3_code(-1.0) == 0
    assert oracle.ue4m3_code(math.inf) == 0


def test_signed_e4m3_round_trip(oracle):
    # format.rs:484-490
    for v in [-448.0, -3.5, -0.25, 0.0, 0.25, 3.5, 448.0]:
        assert oracle.e4m3_value(oracle.e4m3_code(v)) == v
    assert oracle.e4m3_code(math.nan) == 0


def test_tile_layout_offsets(oracle):
    # format.rs:520-527
    assert oracle.scale_layout_len(128, 128) == 1024
    assert oracle.tiled_scale_offset(0, 0, 128) == 0
    assert oracle.tiled_scale_offset(1, 0, 128) == 16
    assert oracle.tiled_scale_offset(32, 0, 128) == 4
    assert oracle.tiled_scale_offset(0, 1, 128) == 1
    assert oracle.tiled_scale_offset(0, 4, 128) == 512


def test_scale_repack(oracle):
    # crates/eider-format/src/modelopt.rs:1323-1330
    src = (np.arange(130 * 5) % 256).astype(np.uint8)
    packed = oracle.scales_to_tiled(src, 130, 80)
    assert packed.size == 2048
    assert packed[0] == src[0]
    assert packed[16] == src[5]
    assert packed[4] == src[32 * 5]


def test_modelopt_k16_encoding(oracle):
    # crates/eider-format/src/modelopt.rs:1281-1294
    row = np.array([[0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0,
                     -6.0]], np.float32)
    packed, scales, g = oracle.quantize_weight(row, global_scale=1.0)
    assert scales.tolist() == [[0x38]]
    assert packed.tolist() == [[0x10, 0x32, 0x54, 0x76, 0x98, 0xBA, 0xDC, 0xFE]]
    deq = oracle.dequantize_weight(packed, scales)
    assert np.array_equal(deq, row)
    assert np.array_equal(np.signbit(deq), np.signbit(row))


def test_quantizes_per_sixteen_value_block(oracle):
    # format.rs:492-503
    values = (np.arange(20, dtype=np.float32) - 10.0).reshape(1, 20)
    packed, scales = oracle.quantize_nvfp4(values)
    assert scales[oracle.tiled_scale_offset(0, 0, 20)] != 0
    assert scales[oracle.tiled_scale_offset(0, 1, 20)] != 0
    assert packed.size == 10


def test_quantizer_fixture_dyadic(oracle):
    # crates/eider-cuda/src/kernels/non_gemm.rs:19655-19683: rows(K)=96, cols(tokens)=3,
    # input_scale=.25, x = ((i % 29) - 14) / 32.  The scaled values are dyadic, so
    # dequantize(quantize(x)) * input_scale lands on representable points.
    k, t = 96, 3
    x = (((np.arange(k * t) % 29) - 14) / 32.0).astype(np.float32).reshape(t, k)
    packed, scales = oracle.quantize_nvfp4(x, input_scale=0.25)
    deq = oracle.dequantize_tiled(packed, scales) * 0.25
    assert scales.size == oracle.scale_layout_len(t, k)
    # block amax/6 rounded to E4M3 keeps |error| within half an E2M1 step of the block scale
    for tok in range(t):
        for b in range(k // 16):
            s = oracle.e4m3_value(int(scales[oracle.tiled_scale_offset(tok, b, k)])) * 0.25
            blk = slice(b * 16, b * 16 + 16)
            assert np.all(np.abs(deq[tok, blk] - x[tok, blk]) <= s * 1.0 + 1e-7)


def test_router_topk_golden(oracle):
    # crates/eider-cuda/src/kernels/non_gemm.rs:17752-17809
    lg = np.array([[0.0, 3.0, 1.0, 2.0]], np.float32)
    for norm in (True, False):
        idx, w = oracle.moe_topk(lg, 2, norm)
        assert idx.tolist() == [[1, 3]]
        if norm:
            assert abs(w.sum() - 1.0) < 1e-6
        else:
            p = np.exp(lg - lg.max())
            p /= p.sum()
            assert np.allclose(w[0], p[0, [1, 3]], atol=1e-6)
    # tie order, non_gemm.rs:17935-17959
    lg = np.full((1, 256), -10.0, np.float32)
    for e in [19, 3, 241, 7, 8, 9, 10, 11, 12]:
        lg[0, e] = 4.0
    idx, w = oracle.moe_topk(lg, 8, True)
    assert idx.tolist() == [[3, 7, 8, 9, 10, 11, 12, 19]]
    assert np.allclose(w, 0.125)


def test_router_all_nonfinite(oracle):
    lg = np.full((1, 8), np.nan, np.float32)
    for norm in (True, False):
        idx, w = oracle.moe_topk(lg, 3, norm)
        assert idx.tolist() == [[0, 1, 2]]
        assert w.tolist() == [[1.0, 0.0, 0.0]]


def test_permute_golden(oracle):
    # crates/eider-cuda/src/kernels/non_gemm.rs:15780-15817
    ind = np.array([3, 1, 3, 0, 1, 2, 3, 2], np.uint32)
    counts, offsets, sorted_routes, sorted_experts, inverse = oracle.moe_sort_routes(ind, 4)
    assert counts.tolist() == [1, 2, 2, 3]
    assert offsets.tolist() == [0, 1, 3, 5, 8]
    assert sorted_experts.tolist() == [0, 1, 1, 2, 2, 3, 3, 3]
    for r in range(8):
        assert sorted_routes[inverse[r]] == r
        assert sorted_experts[inverse[r]] == ind[r]


def test_combine_golden(oracle):
    # crates/eider-cuda/src/kernels/non_gemm.rs:15821-15887
    rows, k, ln = 2, 2, 6
    inverse = np.array([1, 0, 3, 2], np.uint32)
    weights = np.array([0.25, 0.75, 0.4, 0.6], np.float32)
    src = oracle.f32_to_bf16_bits(((np.arange(4 * ln) - 7) / 8.0).astype(np.float32)).reshape(4, ln)
    out = oracle.moe_combine(inverse, weights, src, rows, k)
    srcf = oracle.bf16_bits_to_f32(src)
    for r in range(rows):
        exp = sum(srcf[inverse[r * k + s]] * weights[r * k + s] for s in range(k))
        assert np.allclose(out[r], exp, atol=1e-6)


def test_fp8_fixture(oracle):
    # crates/eider-cuda/src/cublaslt/fp8_tn.rs:303-326: weights cycle [00,30,38,b0,b8],
    # x = ((i % 15) - 7) / 8, s_x = .125, s_w = .03125
    m = n = k = 64
    cyc = np.array([0x00, 0x30, 0x38, 0xB0, 0xB8], np.uint8)
    wq = cyc[np.arange(n * k) % 5].reshape(n, k)
    x = (((np.arange(m * k) % 15) - 7) / 8.0).astype(np.float32).reshape(m, k)
    xq = oracle.quantize_fp8_static(x, 0.125)
    assert np.array_equal(oracle.e4m3_decode(xq) * 0.125, x)  # dyadic: exactly representable
    y = oracle.fp8_linear(xq, np.full(m, 0.125, np.float32), wq, np.full(n, 0.03125, np.float32))
    ref = (x.astype(np.float64) @ (oracle.e4m3_decode(wq).astype(np.float64) * 0.03125).T)
    assert np.allclose(y, ref, rtol=1e-4, atol=1e-4)


def test_gemm_fixture_lcg(oracle):
    # crates/eider-cuda/src/cublaslt/fp4_tn.rs:1465-1542: LCG inputs, quantize both sides,
    # GEMM of the dequantized values; the oracle's own matmul must agree with float64.
    def lcg(seed, count):
        s = seed & 0xFFFFFFFFFFFFFFFF
        out = np.empty(count, np.float32)
        for i in range(count):
            s = (s * 6364136223846793005 + 1442695040888963407) & 0xFFFFFFFFFFFFFFFF
            u = (s >> 40) / float(1 << 24)
            s = (s * 6364136223846793005 + 1442695040888963407) & 0xFFFFFFFFFFFFFFFF
            u2 = (s >> 40) / float(1 << 24)
            out[i] = (2.0 * u - 1.0) * (0.25 + 2.75 * u2)
        return out
    m, n, k = 96, 80, 96
    a = lcg(0x123456789ABCDEF0 ^ m, n * k).reshape(n, k)   # weights [N,K]
    b = lcg(0xFEDCBA9876543210 ^ n, m * k).reshape(m, k)   # tokens  [M,K]
    wp, ws, _ = oracle.quantize_weight(a, global_scale=1.0)
    xp, xs = oracle.quantize_nvfp4(b)
    wd = oracle.dequantize_weight(wp, ws)
    xd = oracle.dequantize_tiled(xp, xs)
    y = oracle.matmul_nt(xd, wd, alpha=0.5)
    ref = 0.5 * (xd.astype(np.float64) @ wd.astype(np.float64).T)
    assert np.all(np.abs(y - ref) <= np.maximum(0.125, 0.01 * np.abs(ref)))
    # the reference's host path (unpack, then f32 matmul) gives the same numbers
    y2 = oracle.nvfp4_linear_host(xd, wp, ws, 0.5)
    assert np.allclose(y2, y, rtol=1e-5, atol=1e-4)


def test_fused_silu_mul_quantize_oracle_is_the_staged_path():
    # non_gemm.cu:559-629 against the staged form: silu-mul in fp32 (same operation order), then the activation quantizer
    from oracle import oracle as o
    rng = np.random.default_rng(3)
    k = 96
    gu = (rng.standard_normal((3, 2 * k)) * 2.0).astype(np.float32)
    packed, scales, act = o.silu_mul_halves_quantize_nvfp4(gu, 0.25, want_act=True)
    g, u = gu[:, :k], gu[:, k:]
    one = np.float32(1.0)
    sig = one / (one + np.exp(-g).astype(np.float32))
    staged = (g * sig).astype(np.float32) * u
    assert np.allclose(act, staged, rtol=2e-6, atol=0)  # numpy's exp may differ from libm's expf in the last place
    p2, s2 = o.quantize_nvfp4(act, 0.25)
    assert np.array_equal(packed, p2) and np.array_equal(scales, s2)
