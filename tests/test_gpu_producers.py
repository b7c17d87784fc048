"""Fused producers of the NVFP4 quantizer against their staged GPU path (byte for byte: the reference's own criterion,
crates/eider-cuda/src/kernels/non_gemm.rs:19687-19750, 19873-20240) and against the CPU oracle; the stand-alone
entry points the staged path is made of; the in-place channel scalings.  Everything goes through the C ABI."""
import numpy as np
import pytest

from tests.util import require_cuda

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


def nvfp4_buffers(rows, cols):
    import torch

    from eider_b200 import ops
    return (torch.zeros(rows, cols // 2, dtype=torch.uint8, device="cuda"),
            torch.zeros(ops.scale_layout_len(rows, cols), dtype=torch.uint8, device="cuda"))


def staged_quantize(lib, values, rows, cols, input_scale):
    """infer_quantize_nvfp4_col_major_f32_on_stream on a device f32 [rows, cols] tensor."""
    p, s = nvfp4_buffers(rows, cols)
    assert lib.infer_quantize_nvfp4_col_major_f32_on_stream(values.data_ptr(), p.data_ptr(), s.data_ptr(), cols, rows, input_scale, None) == 0
    return p, s


def same_bytes(a, b):
    import torch
    torch.cuda.synchronize()
    return torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])


@pytest.mark.parametrize("rows,cols", [(3, 544), (1, 5120), (64, 2048), (5, 12288)])
def test_fused_rms_norm_quantize_equals_staged(lib, rows, cols):
    import torch
    if (rows, cols) == (3, 544):  # the reference's fixture: rows = 3, cols = 544, eps 1e-6, input_scale 0.375
        x = (((np.arange(rows * cols) * 17 % 101).astype(np.float32) - 50.0) * 0.015625).astype(np.float32).reshape(rows, cols)
        w = (0.75 + (np.arange(cols) % 13).astype(np.float32) * 0.03125).astype(np.float32)
    else:
        rng = np.random.default_rng(rows + cols)
        x = (rng.standard_normal((rows, cols)) * np.exp(rng.uniform(-2, 2, (rows, 1)))).astype(np.float32)
        w = rng.uniform(0.5, 1.5, cols).astype(np.float32)
    xd, wd = dev(x), dev(w)
    normed = torch.empty_like(xd)
    assert lib.infer_rms_norm_f32_on_stream(xd.data_ptr(), wd.data_ptr(), normed.data_ptr(), rows, cols, 1e-6, None) == 0
    staged = staged_quantize(lib, normed, rows, cols, 0.375)
    fused = nvfp4_buffers(rows, cols)
    assert lib.infer_rms_norm_quantize_nvfp4_col_major_f32_on_stream(xd.data_ptr(), wd.data_ptr(), fused[0].data_ptr(), fused[1].data_ptr(),
                                                                     rows, cols, 1e-6, 0.375, None) == 0
    assert same_bytes(fused, staged)
    # the staged norm itself against a float64 evaluation
    ref = x.astype(np.float64) / np.sqrt((x.astype(np.float64) ** 2).mean(axis=1, keepdims=True) + 1e-6) * w
    assert np.allclose(normed.cpu().numpy(), ref, rtol=3e-6, atol=1e-7)


@pytest.mark.parametrize("rows,cols", [(3, 96), (1, 5120), (40, 2048)])
def test_fused_add_then_norm_quantize_equals_staged(lib, rows, cols):
    # non_gemm.rs:19873-19960: staged = rms_norm_add_f32, then the fused RMSNorm quantizer on its output
    import torch
    rng = np.random.default_rng(rows * 7 + cols)
    x = rng.standard_normal((rows, cols)).astype(np.float32)
    res = rng.standard_normal((rows, cols)).astype(np.float32)
    w0 = rng.uniform(0.5, 1.5, cols).astype(np.float32)
    w1 = rng.uniform(0.5, 1.5, cols).astype(np.float32)
    xd, rd, w0d, w1d = dev(x), dev(res), dev(w0), dev(w1)
    h_staged = torch.empty_like(xd)
    assert lib.infer_rms_norm_add_f32_on_stream(xd.data_ptr(), w0d.data_ptr(), rd.data_ptr(), h_staged.data_ptr(), rows, cols, 1e-6, None) == 0
    staged = nvfp4_buffers(rows, cols)
    assert lib.infer_rms_norm_quantize_nvfp4_col_major_f32_on_stream(h_staged.data_ptr(), w1d.data_ptr(), staged[0].data_ptr(),
                                                                     staged[1].data_ptr(), rows, cols, 1e-5, 0.375, None) == 0
    # fully staged: norm + add, norm, plain quantizer
    n2 = torch.empty_like(xd)
    assert lib.infer_rms_norm_f32_on_stream(h_staged.data_ptr(), w1d.data_ptr(), n2.data_ptr(), rows, cols, 1e-5, None) == 0
    staged3 = staged_quantize(lib, n2, rows, cols, 0.375)
    h_fused = torch.empty_like(xd)
    fused = nvfp4_buffers(rows, cols)
    assert lib.infer_rms_norm_add_then_rms_norm_quantize_nvfp4_f32_on_stream(
        xd.data_ptr(), w0d.data_ptr(), rd.data_ptr(), h_fused.data_ptr(), w1d.data_ptr(), fused[0].data_ptr(), fused[1].data_ptr(),
        rows, cols, 1e-6, 1e-5, 0.375, None) == 0
    torch.cuda.synchronize()
    assert torch.equal(h_fused, h_staged)
    assert same_bytes(fused, staged) and same_bytes(fused, staged3)


def test_add_then_norm_rejects_rows_beyond_shared_memory(lib):
    import torch
    cols = 12288  # 48 KB of staging plus the kernel's static shared memory does not fit without opting in
    x = torch.zeros(1, cols, device="cuda")
    w = torch.ones(cols, device="cuda")
    p, s = nvfp4_buffers(1, cols)
    assert lib.infer_rms_norm_add_then_rms_norm_quantize_nvfp4_f32_on_stream(
        x.data_ptr(), w.data_ptr(), x.data_ptr(), x.clone().data_ptr(), w.data_ptr(), p.data_ptr(), s.data_ptr(), 1, cols, 1e-6, 1e-6,
        1.0, None) == 1
    cols = 12272
    x = torch.randn(2, cols, device="cuda")
    w = torch.ones(cols, device="cuda")
    out = torch.empty_like(x)
    p, s = nvfp4_buffers(2, cols)
    assert lib.infer_rms_norm_add_then_rms_norm_quantize_nvfp4_f32_on_stream(
        x.data_ptr(), w.data_ptr(), x.data_ptr(), out.data_ptr(), w.data_ptr(), p.data_ptr(), s.data_ptr(), 2, cols, 1e-6, 1e-6, 1.0,
        None) == 0
    torch.cuda.synchronize()


@pytest.mark.parametrize("rows,cols", [(3, 96), (1, 13824), (50, 768)])
def test_fused_gelu_quantize_equals_staged_and_oracle(lib, oracle, rows, cols):
    # non_gemm.rs:20037-20092
    import torch
    if (rows, cols) == (3, 96):
        idx = np.arange(rows * cols)
        gate = (((idx * 17 % 101).astype(np.float32) - 50.0) * 0.015625).astype(np.float32).reshape(rows, cols)
        up = (((idx * 29 % 107).astype(np.float32) - 53.0) * 0.01171875).astype(np.float32).reshape(rows, cols)
    else:
        rng = np.random.default_rng(rows + cols)
        gate = (rng.standard_normal((rows, cols)) * 2).astype(np.float32)
        up = rng.standard_normal((rows, cols)).astype(np.float32)
    gd, ud = dev(gate), dev(up)
    act = torch.empty_like(gd)
    assert lib.infer_gelu_tanh_mul_f32_on_stream(gd.data_ptr(), ud.data_ptr(), act.data_ptr(), rows * cols, None) == 0
    staged = staged_quantize(lib, act, rows, cols, 0.375)
    fused = nvfp4_buffers(rows, cols)
    assert lib.infer_gelu_tanh_mul_quantize_nvfp4_col_major_f32_on_stream(gd.data_ptr(), ud.data_ptr(), fused[0].data_ptr(), fused[1].data_ptr(),
                                                                          rows, cols, 0.375, None) == 0
    assert same_bytes(fused, staged)
    ref = oracle.gelu_tanh_mul(gate, up)
    assert np.allclose(act.cpu().numpy(), ref, rtol=1e-5, atol=2e-6)  # device tanhf against numpy's
    p_ref, s_ref = oracle.quantize_nvfp4(ref, 0.375)
    assert np.count_nonzero(fused[0].cpu().numpy() != p_ref) / p_ref.size < 2e-3
    assert lib.infer_gelu_tanh_mul_quantize_nvfp4_col_major_f32_on_stream(None, ud.data_ptr(), fused[0].data_ptr(), fused[1].data_ptr(),
                                                                          rows, cols, 0.375, None) == 1


@pytest.mark.parametrize("dtype", ["f32", "bf16"])
@pytest.mark.parametrize("tokens,heads,head_dim,offset", [(5, 3, 32, 2), (64, 40, 128, 0)])
def test_fused_head_unpack_quantize_equals_staged_and_oracle(lib, oracle, tokens, heads, head_dim, offset, dtype):
    # non_gemm.rs:20094-20240: rows before the offset stay untouched (zero); bit-exact against the CPU oracle
    import torch
    features = heads * head_dim
    rows = offset + tokens
    idx = np.arange(tokens * features)
    token_major = (((idx * 17 % 101).astype(np.float32) - 50.0) * 0.015625).astype(np.float32).reshape(tokens, heads, head_dim)
    head_major = np.ascontiguousarray(token_major.transpose(1, 0, 2))
    src = dev(head_major, torch.bfloat16 if dtype == "bf16" else None)  # (these values are exact in bf16)
    fused = nvfp4_buffers(rows, features)
    name = f"infer_unpack_heads_quantize_nvfp4_col_major_{dtype}_on_stream"
    assert getattr(lib, name)(src.data_ptr(), fused[0].data_ptr(), fused[1].data_ptr(), tokens, heads, head_dim, offset, 0.375, None) == 0
    unpacked = torch.zeros(rows, features, device="cuda")
    src_f32 = dev(head_major)
    assert lib.infer_unpack_heads_f32_on_stream(src_f32.data_ptr(), unpacked.data_ptr(), tokens, heads, head_dim, offset, None) == 0
    staged = staged_quantize(lib, unpacked, rows, features, 0.375)
    assert same_bytes(fused, staged)
    full = np.zeros((rows, features), np.float32)
    full[offset:] = token_major.reshape(tokens, features)
    assert np.array_equal(unpacked.cpu().numpy(), full)
    p_ref, s_ref = oracle.quantize_nvfp4(full, 0.375)
    assert np.array_equal(fused[0].cpu().numpy(), p_ref) and np.array_equal(fused[1].cpu().numpy(), s_ref)


@pytest.mark.parametrize("rows,heads", [(3, 2), (16, 40)])
def test_fused_gated_rms_norm_quantize_equals_staged(lib, oracle, rows, heads):
    import torch
    cols = heads * 128
    rng = np.random.default_rng(rows + heads)
    x = rng.standard_normal((rows, cols)).astype(np.float32)
    g = (rng.standard_normal((rows, cols)) * 2).astype(np.float32)
    w = rng.uniform(0.5, 1.5, 128).astype(np.float32)
    xd, gd, wd = dev(x), dev(g), dev(w)
    staged_vals = torch.empty_like(xd)
    # per-head norm: the staged operator over rows * heads rows of 128 columns
    assert lib.infer_gated_rms_norm_f32_on_stream(xd.data_ptr(), gd.data_ptr(), wd.data_ptr(), staged_vals.data_ptr(), rows * heads, 128, 1e-6, None) == 0
    staged = staged_quantize(lib, staged_vals, rows, cols, 0.5)
    fused = nvfp4_buffers(rows, cols)
    assert lib.infer_gated_rms_norm_quantize_nvfp4_col_major_f32_on_stream(xd.data_ptr(), gd.data_ptr(), wd.data_ptr(), fused[0].data_ptr(),
                                                                           fused[1].data_ptr(), rows, heads, 128, 1e-6, 0.5, None) == 0
    assert same_bytes(fused, staged)
    xh = x.reshape(rows * heads, 128).astype(np.float64)
    gh = g.reshape(rows * heads, 128).astype(np.float64)
    ref = xh / np.sqrt((xh ** 2).mean(axis=1, keepdims=True) + 1e-6) * w * (gh / (1 + np.exp(-gh)))
    assert np.allclose(staged_vals.cpu().numpy().reshape(-1, 128), ref, rtol=5e-6, atol=1e-6)
    assert lib.infer_gated_rms_norm_quantize_nvfp4_col_major_f32_on_stream(xd.data_ptr(), gd.data_ptr(), wd.data_ptr(), fused[0].data_ptr(),
                                                                           fused[1].data_ptr(), rows, heads, 64, 1e-6, 0.5, None) == 1


@pytest.mark.parametrize("tokens,k", [(1, 768), (33, 2048)])
def test_fused_silu_quantize_against_staged(lib, oracle, tokens, k):
    # The reference spells SiLU differently in its staged kernel ((g / (1 + e^-g)) * u, non_gemm.cu:1369) and in its fused
    # quantizer (g * (1 / (1 + e^-g)) * u, non_gemm.cu:576-577): the two round differently, so here the bar is agreement
    # of the codes up to rare boundary cases, and the staged kernel itself against a float64 evaluation.
    import torch
    rng = np.random.default_rng(tokens + k)
    gu = (rng.standard_normal((tokens, 2 * k)) * 2).astype(np.float32)
    gud = dev(gu)
    act = torch.empty(tokens, k, device="cuda")
    assert lib.infer_silu_mul_halves_f32_batch_on_stream(gud.data_ptr(), act.data_ptr(), tokens, k, None) == 0
    staged = staged_quantize(lib, act, tokens, k, 0.5)
    fused = nvfp4_buffers(tokens, k)
    assert lib.eider_b200_silu_mul_halves_quantize_nvfp4_batch_on_stream(gud.data_ptr(), fused[0].data_ptr(), fused[1].data_ptr(), tokens, k, 0.5, None) == 0
    torch.cuda.synchronize()
    assert (fused[0] != staged[0]).float().mean().item() < 2e-3
    assert (fused[1] != staged[1]).float().mean().item() < 2e-3
    g64, u64 = gu[:, :k].astype(np.float64), gu[:, k:].astype(np.float64)
    assert np.allclose(act.cpu().numpy(), g64 / (1 + np.exp(-g64)) * u64, rtol=2e-6, atol=1e-7)


def test_clamped_silu_halves(lib):
    # crates/eider-cuda/src/ffi.rs:1512, :1527 (kernel non_gemm.cu:1328-1338): gate clamped from above, up from both sides;
    # equals the unclamped kernel on inputs clamped beforehand, bit for bit
    import torch
    rng = np.random.default_rng(4)
    rows, cols, limit = 7, 300, 1.5
    gu = (rng.standard_normal((rows, 2 * cols)) * 3).astype(np.float32)
    gud = dev(gu)
    got = torch.empty(rows, cols, device="cuda")
    assert lib.infer_silu_mul_halves_clamped_f32_batch_on_stream(gud.data_ptr(), got.data_ptr(), rows, cols, limit, None) == 0
    pre = gu.copy()
    pre[:, :cols] = np.minimum(pre[:, :cols], limit)
    pre[:, cols:] = np.clip(pre[:, cols:], -limit, limit)
    pred = dev(pre)
    want = torch.empty(rows, cols, device="cuda")
    assert lib.infer_silu_mul_halves_f32_batch_on_stream(pred.data_ptr(), want.data_ptr(), rows, cols, None) == 0
    one = torch.empty(cols, device="cuda")
    assert lib.infer_silu_mul_halves_clamped_f32_on_stream(gud.data_ptr(), one.data_ptr(), cols, limit, None) == 0
    torch.cuda.synchronize()
    assert torch.equal(got, want) and torch.equal(one, want[0])
    g64, u64 = pre[:, :cols].astype(np.float64), pre[:, cols:].astype(np.float64)
    assert np.allclose(got.cpu().numpy(), g64 / (1 + np.exp(-g64)) * u64, rtol=2e-6, atol=1e-7)
    assert lib.infer_silu_mul_halves_clamped_f32_batch_on_stream(gud.data_ptr(), got.data_ptr(), rows, cols, 0.0, None) == 1
    assert lib.infer_silu_mul_halves_clamped_f32_batch_on_stream(gud.data_ptr(), got.data_ptr(), rows, cols, float("inf"), None) == 1


@pytest.mark.parametrize("rows", [16, 768, 1000, 5])
def test_vector_simple_scales_matches_oracle(lib, oracle, rows):
    import torch
    rng = np.random.default_rng(rows)
    x = (rng.standard_normal(rows) * 3).astype(np.float32)
    blocks = (rows + 15) // 16
    p = torch.zeros((rows + 1) // 2, dtype=torch.uint8, device="cuda")
    s = torch.zeros(blocks, dtype=torch.uint8, device="cuda")
    xd = dev(x)
    assert lib.infer_quantize_nvfp4_vector_simple_scales_f32_on_stream(xd.data_ptr(), p.data_ptr(), s.data_ptr(), rows, 0.25, None) == 0
    torch.cuda.synchronize()
    p_ref, s_ref = oracle.quantize_nvfp4_vector_simple_scales(x, 0.25)
    assert np.array_equal(p.cpu().numpy(), p_ref) and np.array_equal(s.cpu().numpy(), s_ref)
    assert lib.infer_quantize_nvfp4_vector_simple_scales_f32_on_stream(xd.data_ptr(), p.data_ptr(), s.data_ptr(), rows, 0.0, None) == 1


def test_scale_channel_in_place(lib):
    import torch
    rows, channels = 7, 300
    v = torch.randn(rows, channels, device="cuda")
    cs = torch.rand(channels, device="cuda") + 0.5
    rs = torch.rand(rows, device="cuda") + 0.5
    want = v * (cs[None, :] * rs[:, None])
    got = v.clone()
    assert lib.infer_scale_channel_f32_device_row_scalar_on_stream(got.data_ptr(), cs.data_ptr(), rs.data_ptr(), rows, channels, None) == 0
    torch.cuda.synchronize()
    assert torch.equal(got, want)
    one = v[0].clone()
    scalar = torch.tensor([0.375], device="cuda")
    assert lib.infer_scale_channel_f32_device_scalar_on_stream(one.data_ptr(), cs.data_ptr(), scalar.data_ptr(), channels, None) == 0
    torch.cuda.synchronize()
    assert torch.equal(one, v[0] * (cs * scalar))
    assert lib.infer_scale_channel_f32_device_scalar_on_stream(None, cs.data_ptr(), scalar.data_ptr(), channels, None) == 1
