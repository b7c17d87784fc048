"""Bit-exact parity of the CUDA quantizers against the CPU oracle (through the C ABI)."""
import math

import numpy as np
import pytest

from tests.test_oracle_golden import E2M1_VALUES
from tests.util import require_cuda

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


def test_reference_fixture_static_scale(ops, oracle):
    # crates/eider-cuda/src/kernels/non_gemm.rs:19655-19683: K=96, 3 tokens, input_scale=.25
    k, t = 96, 3
    x = (((np.arange(k * t) % 29) - 14) / 32.0).astype(np.float32).reshape(t, k)
    q = ops.quantize_nvfp4(_dev(x), 0.25)
    packed, scales = oracle.quantize_nvfp4(x, 0.25)
    assert np.array_equal(q.packed.cpu().numpy(), packed)
    assert np.array_equal(q.scales.cpu().numpy(), scales)


@pytest.mark.parametrize("tokens,k", [(1, 16), (1, 5120), (7, 544), (130, 2048), (512, 5120)])
@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_static_scale_random(ops, oracle, tokens, k, dtype):
    import torch
    rng = np.random.default_rng(tokens * 1000 + k)
    x = rng.standard_normal((tokens, k)).astype(np.float32) * np.exp(rng.uniform(-3, 3, (tokens, 1))).astype(np.float32)
    if dtype == "bf16":
        x = oracle.bf16_round(x)
    xd = _dev(x, torch.bfloat16 if dtype == "bf16" else None)
    for scale in (1.0, 0.37):
        q = ops.quantize_nvfp4(xd, scale)
        packed, scales = oracle.quantize_nvfp4(x, scale)
        assert np.array_equal(q.packed.cpu().numpy(), packed)
        assert np.array_equal(q.scales.cpu().numpy(), scales)


def test_edge_values(ops, oracle):
    # every tie point / saturation / NaN / signed zero of the reference's E2M1 list, one per block position
    vals = np.array(E2M1_VALUES, np.float32)
    pad = (-len(vals)) % 16
    x = np.concatenate([vals, np.zeros(pad, np.float32)]).reshape(1, -1)
    # block scale 1.0: put a 6.0 in every block so the codes are the raw E2M1 roundings
    x = x.reshape(-1, 16).copy()
    x = np.concatenate([x[:, :15], np.full((x.shape[0], 1), 6.0, np.float32)], axis=1).reshape(1, -1)
    q = ops.quantize_nvfp4(_dev(x), 1.0)
    packed, scales = oracle.quantize_nvfp4(x, 1.0)
    assert np.array_equal(q.packed.cpu().numpy(), packed)
    assert np.array_equal(q.scales.cpu().numpy(), scales)


def test_all_zero_and_nonfinite_rows(ops, oracle):
    x = np.zeros((3, 64), np.float32)
    x[1, 5] = np.inf
    x[1, 6] = 2.0
    x[2, 17] = np.nan
    x[2, 18] = -3.0
    q = ops.quantize_nvfp4(_dev(x), 1.0)
    packed, scales = oracle.quantize_nvfp4(x, 1.0)
    assert np.array_equal(q.packed.cpu().numpy(), packed)
    assert np.array_equal(q.scales.cpu().numpy(), scales)
    qr = ops.quantize_nvfp4_rowscale(_dev(x))
    p2, s2, r2 = oracle.quantize_nvfp4_rowscale(x)
    assert np.array_equal(qr.packed.cpu().numpy(), p2)
    assert np.array_equal(qr.scales.cpu().numpy(), s2)
    assert np.array_equal(qr.row_scales.cpu().numpy(), r2)


# (up to 16384 elements per row: one thread per 16-element block; up to 32768: one thread per 8 elements in up to four
# passes; longer rows: the generic kernel)
@pytest.mark.parametrize("tokens,k", [(1, 5120), (33, 2048), (512, 5120), (130, 13824), (3, 8208), (5, 32768), (2, 32784),
                                      (1300, 13824)])
@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_rowscale(ops, oracle, tokens, k, dtype):
    import torch
    rng = np.random.default_rng(7 + tokens)
    x = rng.standard_normal((tokens, k)).astype(np.float32)
    if dtype == "bf16":
        x = oracle.bf16_round(x)
    q = ops.quantize_nvfp4_rowscale(_dev(x, torch.bfloat16 if dtype == "bf16" else None))
    packed, scales, row = oracle.quantize_nvfp4_rowscale(x)
    assert np.array_equal(q.row_scales.cpu().numpy(), row)
    assert np.array_equal(q.packed.cpu().numpy(), packed)
    assert np.array_equal(q.scales.cpu().numpy(), scales)


@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_rowscale_with_specials_everywhere(ops, oracle, dtype):
    # signed zeros, infinities of both signs, NaNs, denormals and huge values sprinkled over random rows: blocks with an
    # infinity take the kernel's careful path, all others the short one, and both must give the reference's bytes
    import torch
    rng = np.random.default_rng(11)
    tokens, k = 96, 5120
    x = rng.standard_normal((tokens, k)).astype(np.float32)
    x[rng.random((tokens, k)) < 0.02] = 0.0
    x[rng.random((tokens, k)) < 0.02] = -0.0
    x[rng.random((tokens, k)) < 0.002] = np.inf
    x[rng.random((tokens, k)) < 0.002] = -np.inf
    x[rng.random((tokens, k)) < 0.002] = np.nan
    x[rng.random((tokens, k)) < 0.01] *= 1e-30
    x[5] *= 1e20
    x[6] *= 1e-25
    x[7, :] = 0.0
    x[8, :16] = -0.0
    x[9, 16:32] = [np.inf] * 8 + [-np.inf] * 8
    if dtype == "bf16":
        x = oracle.bf16_round(x)
    q = ops.quantize_nvfp4_rowscale(_dev(x, torch.bfloat16 if dtype == "bf16" else None))
    packed, scales, row = oracle.quantize_nvfp4_rowscale(x)
    assert np.array_equal(q.row_scales.cpu().numpy(), row)
    assert np.array_equal(q.scales.cpu().numpy(), scales)
    assert np.array_equal(q.packed.cpu().numpy(), packed)


def test_weight_quantize_and_repack(ops, oracle):
    rng = np.random.default_rng(3)
    w = (rng.standard_normal((384, 1024)) * 0.02).astype(np.float32)
    wd = ops.ModelOptWeight.quantize(_dev(w))
    packed, scales, g = oracle.quantize_weight(w)
    assert wd.weight_scale_2 == float(g)
    assert np.array_equal(wd.packed.cpu().numpy(), packed)
    assert np.array_equal(wd.scales_row_major.cpu().numpy(), scales)
    assert np.array_equal(wd.scales_tiled.cpu().numpy(), oracle.scales_to_tiled(scales, 384, 1024))


def test_modelopt_k16_known_answer(ops):
    # crates/eider-format/src/modelopt.rs:1281-1294
    row = np.array([[0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0]], np.float32)
    wd = ops.ModelOptWeight.quantize(_dev(row), global_scale=1.0)
    assert wd.scales_row_major.cpu().numpy().tolist() == [[0x38]]
    assert wd.packed.cpu().numpy().tolist() == [[0x10, 0x32, 0x54, 0x76, 0x98, 0xBA, 0xDC, 0xFE]]


def test_invalid_arguments(ops):
    import torch
    x = torch.zeros(2, 32, device="cuda")
    with pytest.raises(ops.ShapeError):
        ops.quantize_nvfp4(x, 0.0)
    from eider_b200 import _lib
    lib = _lib.load()
    assert lib.infer_quantize_nvfp4_col_major_f32_on_stream(None, None, None, 16, 1, 1.0, None) == 1  # cudaErrorInvalidValue
    assert lib.infer_quantize_nvfp4_col_major_f32_on_stream(x.data_ptr(), x.data_ptr(), x.data_ptr(), 0, 1, 1.0, None) == 1
    assert lib.infer_quantize_nvfp4_col_major_f32_on_stream(x.data_ptr(), x.data_ptr(), x.data_ptr(), 16, 1, math.inf, None) == 1


@pytest.mark.parametrize("rows,cols", [(1, 5120), (8, 5120), (64, 1000)])
@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_fp8_dynamic(ops, oracle, rows, cols, dtype):
    import torch
    rng = np.random.default_rng(rows + cols)
    x = rng.standard_normal((rows, cols)).astype(np.float32)
    if dtype == "bf16":
        x = oracle.bf16_round(x)
    q, s = ops.quantize_fp8_dynamic(_dev(x, torch.bfloat16 if dtype == "bf16" else None))
    qo, so = oracle.quantize_fp8_dynamic(x)
    assert np.array_equal(s.cpu().numpy(), so)
    assert np.array_equal(q.cpu().numpy(), qo)


def test_fp8_static_and_weight(ops, oracle):
    rng = np.random.default_rng(11)
    x = rng.standard_normal((5, 4100)).astype(np.float32)
    q = ops.quantize_fp8_static(_dev(x), 0.125)
    assert np.array_equal(q.cpu().numpy(), oracle.quantize_fp8_static(x, 0.125))
    w = (rng.standard_normal((96, 512)) * 0.02).astype(np.float32)
    wq, ws = ops.quantize_fp8_weight(_dev(w))
    wqo, wso = oracle.quantize_fp8_weight(w)
    assert np.array_equal(ws.cpu().numpy(), wso)
    assert np.array_equal(wq.cpu().numpy(), wqo)


@pytest.mark.parametrize("tokens,k,scale", [(1, 768, 1.0), (1, 13824, 0.03125), (5, 2048, 1.0), (130, 256, 0.5)])
def test_fused_silu_mul_quantize_matches_oracle(ops, oracle, tokens, k, scale):
    # non_gemm.cu:559-629: value = g * (1 / (1 + expf(-g))) * up / input_scale, then the block quantizer; the device's
    # expf may differ from the host's in the last place, which can move a code across a rounding boundary now and then
    import torch
    rng = np.random.default_rng(tokens + k)
    gu = (rng.standard_normal((tokens, 2 * k)) * 2.0).astype(np.float32)
    gu[0, :16] = 0.0  # an all-zero block: scale byte 0, codes 0
    q = ops.silu_mul_halves_quantize_nvfp4(torch.from_numpy(gu).cuda(), scale)
    torch.cuda.synchronize()
    p_ref, s_ref, act = oracle.silu_mul_halves_quantize_nvfp4(gu, scale, want_act=True)
    got_p, got_s = q.packed.cpu().numpy(), q.scales.cpu().numpy()
    assert np.count_nonzero(got_p != p_ref) / got_p.size < 2e-3
    assert np.count_nonzero(got_s != s_ref) / got_s.size < 2e-3
    deq = oracle.dequantize_tiled(got_p, got_s) * scale
    bmax = np.abs(act).reshape(tokens, -1, 16).max(axis=2).repeat(16, axis=1)
    assert np.all(np.abs(deq - act) <= 0.27 * bmax + 1e-12)
    if tokens == 1:  # the reference's single-token entry point gives the same bytes
        from eider_b200 import _lib
        lib = _lib.load()
        p1 = torch.zeros(k // 2, dtype=torch.uint8, device="cuda")
        s1 = torch.zeros_like(q.scales)
        assert lib.infer_silu_mul_halves_quantize_nvfp4_col_major_f32_on_stream(
            torch.from_numpy(gu).cuda().data_ptr(), p1.data_ptr(), s1.data_ptr(), k, scale, None) == 0
        torch.cuda.synchronize()
        assert np.array_equal(p1.cpu().numpy(), got_p[0]) and np.array_equal(s1.cpu().numpy(), got_s)
        assert lib.infer_silu_mul_halves_quantize_nvfp4_col_major_f32_on_stream(None, p1.data_ptr(), s1.data_ptr(), k, scale, None) == 1


@pytest.mark.parametrize("rows,cols,scale", [(1, 5120, 1.0), (7, 2048, 0.25), (300, 256, 1.0)])
def test_fused_rms_norm_quantize_matches_oracle(ops, oracle, rows, cols, scale):
    # non_gemm.cu:193-288: x * rsqrt(mean(x^2) + eps) * weight / input_scale, then the block quantizer.  The sum of
    # squares has no canonical order (and the device uses rsqrtf), so inverse_rms may differ from the oracle's by an
    # ulp or two, which moves a code across a rounding boundary now and then.
    import torch
    rng = np.random.default_rng(rows + cols)
    x = (rng.standard_normal((rows, cols)) * np.exp(rng.uniform(-1, 1, (rows, 1)))).astype(np.float32)
    w = rng.uniform(0.5, 1.5, cols).astype(np.float32)
    q = ops.rms_norm_quantize_nvfp4(torch.from_numpy(x).cuda(), torch.from_numpy(w).cuda(), 1e-6, scale)
    torch.cuda.synchronize()
    p_ref, s_ref, norm = oracle.rms_norm_quantize_nvfp4(x, w, 1e-6, scale, want_norm=True)
    got_p, got_s = q.packed.cpu().numpy(), q.scales.cpu().numpy()
    assert np.count_nonzero(got_p != p_ref) / got_p.size < 5e-3
    assert np.count_nonzero(got_s != s_ref) / got_s.size < 5e-3
    deq = oracle.dequantize_tiled(got_p, got_s)
    bmax = np.abs(norm).reshape(rows, -1, 16).max(axis=2).repeat(16, axis=1)
    assert np.all(np.abs(deq - norm) <= 0.27 * bmax + 1e-12)
    from eider_b200 import _lib
    assert _lib.load().infer_rms_norm_quantize_nvfp4_col_major_f32_on_stream(None, None, None, None, rows, cols, 1e-6, scale, None) == 1


@pytest.mark.parametrize("rows,cols", [(1, 5120), (9, 2048), (200, 256)])
def test_fused_add_then_norm_quantize_matches_oracle(ops, oracle, rows, cols):
    # non_gemm.cu:746-870: h = rmsnorm(x) * w0 + residual (stored), then the quantizing RMSNorm of h
    import torch
    rng = np.random.default_rng(rows * 3 + cols)
    x = rng.standard_normal((rows, cols)).astype(np.float32)
    res = rng.standard_normal((rows, cols)).astype(np.float32)
    w0 = rng.uniform(0.5, 1.5, cols).astype(np.float32)
    w1 = rng.uniform(0.5, 1.5, cols).astype(np.float32)
    dev = lambda a: torch.from_numpy(a).cuda()
    h, q = ops.rms_norm_add_then_rms_norm_quantize_nvfp4(dev(x), dev(w0), dev(res), dev(w1), 1e-6, 1e-5, 0.5)
    torch.cuda.synchronize()
    h_ref, p_ref, s_ref, norm = oracle.rms_norm_add_then_rms_norm_quantize_nvfp4(x, w0, res, w1, 1e-6, 1e-5, 0.5)
    assert np.allclose(h.cpu().numpy(), h_ref, rtol=2e-6, atol=2e-6)
    got_p, got_s = q.packed.cpu().numpy(), q.scales.cpu().numpy()
    assert np.count_nonzero(got_p != p_ref) / got_p.size < 5e-3
    assert np.count_nonzero(got_s != s_ref) / got_s.size < 5e-3
    deq = oracle.dequantize_tiled(got_p, got_s)
    bmax = np.abs(norm).reshape(rows, -1, 16).max(axis=2).repeat(16, axis=1)
    assert np.all(np.abs(deq - norm) <= 0.27 * bmax + 1e-12)


@pytest.mark.parametrize("rows,cols", [(1, 5120), (33, 1024)])
def test_fused_rms_norm_quantize_pair_matches_oracle(ops, oracle, rows, cols):
    # non_gemm.cu:290-419: the second term quantizes what the first left, block by block
    import torch
    from eider_b200 import _lib
    lib = _lib.load()
    rng = np.random.default_rng(rows + cols + 1)
    x = rng.standard_normal((rows, cols)).astype(np.float32)
    w = rng.uniform(0.5, 1.5, cols).astype(np.float32)
    xd, wd = torch.from_numpy(x).cuda(), torch.from_numpy(w).cuda()
    n_sf = oracle.scale_layout_len(rows, cols)
    p = torch.zeros(rows, cols // 2, dtype=torch.uint8, device="cuda")
    rp = torch.zeros_like(p)
    s_ = torch.zeros(n_sf, dtype=torch.uint8, device="cuda")
    rs = torch.zeros_like(s_)
    assert lib.infer_rms_norm_quantize_nvfp4_pair_col_major_f32_on_stream(xd.data_ptr(), wd.data_ptr(), p.data_ptr(), s_.data_ptr(),
                                                                          rp.data_ptr(), rs.data_ptr(), rows, cols, 1e-6, 1.0, None) == 0
    torch.cuda.synchronize()
    p0, s0, rp0, rs0 = oracle.rms_norm_quantize_nvfp4_pair(x, w, 1e-6, 1.0)
    _, _, norm = oracle.rms_norm_quantize_nvfp4(x, w, 1e-6, 1.0, want_norm=True)
    got = [t.cpu().numpy() for t in (p, s_, rp, rs)]
    for a, b in zip(got, (p0, s0, rp0, rs0)):
        assert np.count_nonzero(a != b) / a.size < 1e-2
    # the first term alone equals the single-term producer bit for bit
    q1 = ops.rms_norm_quantize_nvfp4(xd, wd, 1e-6, 1.0)
    assert torch.equal(q1.packed, p) and torch.equal(q1.scales, s_)
    two = oracle.dequantize_tiled(got[0], got[1]) + oracle.dequantize_tiled(got[2], got[3])
    bmax = np.abs(norm).reshape(rows, -1, 16).max(axis=2).repeat(16, axis=1)
    assert np.all(np.abs(two - norm) <= 0.08 * bmax + 1e-12)
