"""tcgen05 GEMMs against the oracle: GPU result vs host dequantize + fp32-accumulated matmul, the reference's own
criterion (crates/eider-cuda/src/cublaslt/fp4_tn.rs:1503-1542, fp8_tn.rs:303-362)."""
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


def _lcg(seed, count):
    # crates/eider-cuda/src/cublaslt/fp4_tn.rs:1465-1510
    s = seed & 0xFFFFFFFFFFFFFFFF
    out = np.empty(count, np.float32)
    for i in range(count):
        s = (s * 6364136223846793005 + 1442695040888963407) & 0xFFFFFFFFFFFFFFFF
        u = (s >> 40) / float(1 << 24)
        s = (s * 6364136223846793005 + 1442695040888963407) & 0xFFFFFFFFFFFFFFFF
        u2 = (s >> 40) / float(1 << 24)
        out[i] = (2.0 * u - 1.0) * (0.25 + 2.75 * u2)
    return out


def _nvfp4_case(ops, oracle, x, w, block_n=None, rowscale=False, out_dtype="f32", alpha=None, beta=0.0, splits=None):
    import torch
    m, k = x.shape
    n = w.shape[0]
    wp, ws, g = oracle.quantize_weight(w)
    wd = ops.ModelOptWeight.from_checkpoint(_dev(wp), _dev(ws), float(g))
    if rowscale:
        xq = ops.quantize_nvfp4_rowscale(_dev(x))
        xp, xs, xr = oracle.quantize_nvfp4_rowscale(x)
    else:
        xq = ops.quantize_nvfp4(_dev(x), 1.0)
        xp, xs = oracle.quantize_nvfp4(x, 1.0)
        xr = None
    assert np.array_equal(xq.packed.cpu().numpy(), xp)
    assert np.array_equal(xq.scales.cpu().numpy(), xs)
    plan = ops.Fp4TnMatmulPlan(m, n, k)
    if block_n:
        plan.set_block_n(block_n)
    if splits is not None:
        plan.set_k_splits(splits)  # (after the tile shape: setting that one lets the plan choose its own split count again)
        assert plan.k_splits == splits
    dt = torch.float32 if out_dtype == "f32" else torch.bfloat16
    a = float(g) if alpha is None else alpha
    rng = np.random.default_rng(1)
    c0 = rng.standard_normal((m, n)).astype(np.float32)
    if out_dtype != "f32":
        c0 = oracle.bf16_round(c0)
    out = _dev(c0, dt) if beta != 0.0 else torch.full((m, n), float("nan"), dtype=dt, device="cuda")
    plan.run(xq, wd, out=out, alpha=a, beta=beta)
    torch.cuda.synchronize()
    assert plan.status() == 0
    ref = oracle.matmul_nt(oracle.dequantize_tiled(xp, xs), oracle.dequantize_weight(wp, ws), alpha=a, row_scale=xr)
    if beta != 0.0:
        ref = ref + beta * c0
    got = to_np(out)
    assert not np.isnan(got).any()
    ok, stats = gemm_close(got, ref)
    assert ok, stats
    return stats


@pytest.mark.parametrize("m,n,k", [(64, 64, 64), (128, 128, 128), (96, 80, 96)])
def test_reference_fixture_shapes(ops, oracle, m, n, k):
    # fp4_tn.rs:1503-1650: 64^3, 128^3 and the partial-tile 96x80x96 case, LCG inputs, tol max(0.125, 1 %)
    w = _lcg(0x123456789ABCDEF0 ^ m, n * k).reshape(n, k)
    x = _lcg(0xFEDCBA9876543210 ^ n, m * k).reshape(m, k)
    _nvfp4_case(ops, oracle, x, w)


def test_all_ones_is_exact(ops):
    # crates/eider-cuda/src/diagnostics/smoke.rs:34-64: E2M1 ones (code 0x2) with unit scales (0x38), 128^3,
    # must give exactly 128
    import torch
    packed = torch.full((128, 64), 0x22, dtype=torch.uint8, device="cuda")
    scales_rm = torch.full((128, 8), 0x38, dtype=torch.uint8, device="cuda")
    wd = ops.ModelOptWeight.from_checkpoint(packed, scales_rm, 1.0)
    xq = ops.Nvfp4Matrix(packed.clone(), wd.scales_tiled.clone(), 128, 128)
    y = ops.Fp4TnMatmulPlan(128, 128, 128).run(xq, wd, out_dtype=torch.float32)
    assert np.all(to_np(y) == 128.0)


@pytest.mark.parametrize("block_n", [64, 128, 256])
@pytest.mark.parametrize("m,n,k", [(1, 16, 32), (130, 264, 1056), (512, 1024, 5120), (300, 5120, 13824)])
def test_nvfp4_gemm_random(ops, oracle, m, n, k, block_n):
    rng = np.random.default_rng(m + n + k)
    x = rng.standard_normal((m, k)).astype(np.float32)
    w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    _nvfp4_case(ops, oracle, x, w, block_n=block_n, rowscale=True, out_dtype="bf16")


@pytest.mark.parametrize("block_n", [512, 384])
@pytest.mark.parametrize("m,n,k", [(256, 256, 256), (130, 264, 1056), (384, 640, 288), (512, 1024, 5120), (1000, 2304, 2048), (512, 3456, 512)])
def test_nvfp4_gemm_cta_pairs(ops, oracle, m, n, k, block_n):
    # tile code 512: 256 x 256 tiles computed by clusters of two CTAs (tcgen05 cta_group::2), 384: 256 x 192 tiles (two whole
    # accumulators, every other tile starting in the middle of a 128-row scale tile); odd row-tile counts, partial tiles in
    # both directions and a K that is not a multiple of the stage depth are all in the list
    rng = np.random.default_rng(m * 7 + n + k)
    x = rng.standard_normal((m, k)).astype(np.float32)
    w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    _nvfp4_case(ops, oracle, x, w, block_n=block_n, rowscale=True, out_dtype="bf16")


def test_nvfp4_gemm_cta_pairs_general_epilogue(ops, oracle):
    # fp32 output and beta * C go through the element-wise epilogue of the pair kernel
    rng = np.random.default_rng(11)
    x = rng.standard_normal((300, 512)).astype(np.float32)
    w = rng.standard_normal((328, 512)).astype(np.float32)
    for code in (512, 384):
        _nvfp4_case(ops, oracle, x, w, block_n=code, out_dtype="f32")
        _nvfp4_case(ops, oracle, x, w, block_n=code, beta=0.5, out_dtype="bf16", alpha=0.01)


def test_nvfp4_gemm_beta_accumulate(ops, oracle):
    # D = alpha * X.W^T + beta * C with C = D in place (fp4_tn.rs:603-678, residual add fused with beta = 1)
    rng = np.random.default_rng(5)
    x = rng.standard_normal((140, 512)).astype(np.float32)
    w = rng.standard_normal((200, 512)).astype(np.float32)
    _nvfp4_case(ops, oracle, x, w, beta=1.0, out_dtype="f32")
    _nvfp4_case(ops, oracle, x, w, beta=0.5, out_dtype="bf16", alpha=0.01)


def test_nvfp4_gemm_linearity_full_size(ops):
    # size-independent property at the benchmark shape: doubling alpha doubles the bf16-rounded result exactly
    import torch
    m, n, k = 512, 27648, 5120
    g = torch.Generator(device="cuda").manual_seed(0)
    w = torch.randn(n, k, device="cuda", generator=g) * 0.02
    x = torch.randn(m, k, device="cuda", generator=g).to(torch.bfloat16)
    wd = ops.ModelOptWeight.quantize(w)
    del w
    xq = ops.quantize_nvfp4_rowscale(x)
    plan = ops.Fp4TnMatmulPlan(m, n, k)
    y1 = plan.run(xq, wd)
    y2 = plan.run(xq, wd, alpha=2.0 * wd.matmul_alpha)
    torch.cuda.synchronize()
    assert plan.status() == 0
    assert torch.equal(y2.float(), 2.0 * y1.float())
    assert torch.isfinite(y1.float()).all()  # (element-wise parity at this shape: test_gpu_full_size.py)


def test_fp8_fixture(ops, oracle):
    # crates/eider-cuda/src/cublaslt/fp8_tn.rs:303-326: M=K=256, weights cycle [00,30,38,b0,b8], x=((i%15)-7)/8
    m = n = k = 256
    cyc = np.array([0x00, 0x30, 0x38, 0xB0, 0xB8], np.uint8)
    wq = cyc[np.arange(n * k) % 5].reshape(n, k)
    x = (((np.arange(m * k) % 15) - 7) / 8.0).astype(np.float32).reshape(m, k)
    xq = oracle.quantize_fp8_static(x, 0.125)
    import torch
    plan = ops.Fp8TnMatmulPlan(m, n, k)
    y = plan.run(_dev(xq), _dev(wq), None, None, alpha=0.125 * 0.03125, out_dtype=torch.float32)
    ref = oracle.fp8_linear(xq, np.full(m, 0.125, np.float32), wq, np.full(n, 0.03125, np.float32))
    assert plan.status() == 0
    assert np.allclose(to_np(y), ref, rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("m,n,k", [(1, 7168, 5120), (8, 7168, 5120), (64, 1000, 528), (200, 328, 1040)])
def test_fp8_gemm_scaled(ops, oracle, m, n, k):
    import torch
    rng = np.random.default_rng(m + n)
    w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    x = oracle.bf16_round(rng.standard_normal((m, k)).astype(np.float32))
    wq, ws = ops.quantize_fp8_weight(_dev(w))
    xq, xs = ops.quantize_fp8_dynamic(_dev(x, torch.bfloat16))
    wqo, wso = oracle.quantize_fp8_weight(w)
    xqo, xso = oracle.quantize_fp8_dynamic(x)
    assert np.array_equal(wq.cpu().numpy(), wqo) and np.array_equal(xq.cpu().numpy(), xqo)
    plan = ops.Fp8TnMatmulPlan(m, n, k)
    y = plan.run(xq, wq, xs, ws, out_dtype=torch.bfloat16)
    assert plan.status() == 0
    ref = oracle.fp8_linear(xqo, xso, wqo, wso)
    ok, stats = gemm_close(to_np(y), ref)
    assert ok, stats


@pytest.mark.parametrize("block_n", [512, 384])
@pytest.mark.parametrize("m,n,k", [(256, 512, 1024), (300, 328, 1040)])
def test_fp8_gemm_cta_pairs(ops, oracle, m, n, k, block_n):
    import torch
    rng = np.random.default_rng(m + n + 1)
    w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    x = oracle.bf16_round(rng.standard_normal((m, k)).astype(np.float32))
    wq, ws = ops.quantize_fp8_weight(_dev(w))
    xq, xs = ops.quantize_fp8_dynamic(_dev(x, torch.bfloat16))
    plan = ops.Fp8TnMatmulPlan(m, n, k)
    plan.set_block_n(block_n)
    y = plan.run(xq, wq, xs, ws, out_dtype=torch.bfloat16)
    assert plan.status() == 0
    ref = oracle.fp8_linear(xq.cpu().numpy(), xs.cpu().numpy(), wq.cpu().numpy(), ws.cpu().numpy())
    ok, stats = gemm_close(to_np(y), ref)
    assert ok, stats


@pytest.mark.parametrize("m,n,k,block_n,splits", [(128, 320, 4096, 128, 3), (100, 264, 2080, 64, 2), (128, 512, 4096, 256, 2),
                                                   (256, 512, 4096, 512, 4), (300, 328, 2336, 512, 2), (40, 5120, 13824, 128, 3),
                                                   (300, 400, 2336, 384, 3)])
@pytest.mark.parametrize("out_dtype,beta,rowscale", [("bf16", 0.0, True), ("f32", 0.5, False)])
def test_nvfp4_gemm_split_k(ops, oracle, m, n, k, block_n, splits, out_dtype, beta, rowscale):
    # K divided over several work items per tile, fp32 partial sums summed by a second kernel: same criterion as unsplit
    rng = np.random.default_rng(m + n + k + splits)
    x = rng.standard_normal((m, k)).astype(np.float32)
    w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    _nvfp4_case(ops, oracle, x, w, block_n=block_n, rowscale=rowscale, out_dtype=out_dtype, beta=beta, splits=splits)


@pytest.mark.parametrize("block_n,splits", [(128, 3), (512, 2)])
def test_fp8_gemm_split_k(ops, oracle, block_n, splits):
    import torch
    m, n, k = 200, 328, 2064
    rng = np.random.default_rng(7)
    w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    x = oracle.bf16_round(rng.standard_normal((m, k)).astype(np.float32))
    wq, ws = ops.quantize_fp8_weight(_dev(w))
    xq, xs = ops.quantize_fp8_dynamic(_dev(x, torch.bfloat16))
    plan = ops.Fp8TnMatmulPlan(m, n, k)
    plan.set_block_n(block_n)
    plan.set_k_splits(splits)
    y = plan.run(xq, wq, xs, ws, out_dtype=torch.bfloat16)
    assert plan.status() == 0
    ref = oracle.fp8_linear(xq.cpu().numpy(), xs.cpu().numpy(), wq.cpu().numpy(), ws.cpu().numpy())
    ok, stats = gemm_close(to_np(y), ref)
    assert ok, stats


def test_split_k_choice_and_argument_checks(ops):
    from eider_b200._lib import CudaError
    # few tiles and a long K: split; enough tiles, or a short K: not
    assert ops.Fp4TnMatmulPlan(128, 2560, 13824).k_splits == 3
    narrow = ops.Fp4TnMatmulPlan(128, 5120, 13824)  # 80 tiles of 64 weight rows: no split would fit in one wave
    assert narrow.block_n == 64 and narrow.k_splits == 1
    assert ops.Fp4TnMatmulPlan(384, 27648, 5120).block_n == 192
    assert ops.Fp4TnMatmulPlan(512, 27648, 5120).k_splits == 1
    assert ops.Fp4TnMatmulPlan(128, 27648, 5120).k_splits == 1
    assert ops.Fp4TnMatmulPlan(4096, 5120, 13824).k_splits == 1
    assert ops.Fp4TnMatmulPlan(256, 5120, 13824).k_splits == 1  # (more than one row tile: the partial sums cost more than they save)
    # tile shape: pairs of CTAs from two row tiles on; 256 x 192 tiles where they save a turn of the 74 SM pairs
    assert ops.Fp4TnMatmulPlan(512, 27648, 5120).block_n == 512
    assert ops.Fp4TnMatmulPlan(4096, 27648, 5120).block_n == 512
    assert ops.Fp4TnMatmulPlan(512, 5120, 13824).block_n == 384
    assert ops.Fp4TnMatmulPlan(1024, 5120, 13824).block_n == 384
    assert ops.Fp4TnMatmulPlan(8192, 5120, 13824).block_n == 512
    plan = ops.Fp4TnMatmulPlan(128, 256, 512)  # two 128-byte K stages
    for bad in (0, 17, 3):
        with pytest.raises(CudaError):
            plan.set_k_splits(bad)
    plan.set_k_splits(2)
    assert plan.k_splits == 2


def test_gemm_rejects_bad_arguments(ops):
    from eider_b200 import _lib
    lib = _lib.load()
    assert lib.eider_b200_nvfp4_gemm_tn_supported(128, 128, 48) == 0
    assert lib.eider_b200_nvfp4_gemm_tn_supported(0, 128, 64) == 0
    assert not lib.eider_b200_nvfp4_gemm_tn_create(128, 128, 40)
    with pytest.raises(ops.ShapeError):
        ops.Fp4TnMatmulPlan(16, 16, 24)
    plan = lib.eider_b200_nvfp4_gemm_tn_create(128, 128, 128)
    assert lib.eider_b200_nvfp4_gemm_tn_on_stream(plan, None, None, None, None, None, None, 1.0, 0.0, None, 1, None) == 1
    lib.eider_b200_nvfp4_gemm_tn_destroy(plan)


def test_dense_ffn_composition(ops, oracle):
    # gate_up -> SiLU * up -> quantize -> down + residual -> bf16 (crates/infer/src/qwen3/qwen36.rs:7175-7280), stage by stage
    # against the oracle, with the plan cache keyed by row count
    import torch
    hidden, inter = 1024, 768
    rng = np.random.default_rng(4)
    wgu = (rng.standard_normal((2 * inter, hidden)) * 0.02).astype(np.float32)
    wdn = (rng.standard_normal((hidden, inter)) * 0.02).astype(np.float32)
    gp, gs, gg = oracle.quantize_weight(wgu)
    dp, ds, dg = oracle.quantize_weight(wdn)
    in_scale = 0.015625
    ffn = ops.DenseFfn(ops.ModelOptWeight.from_checkpoint(_dev(gp), _dev(gs), float(gg)),
                       ops.ModelOptWeight.from_checkpoint(_dev(dp), _dev(ds), float(dg), input_scale=in_scale))
    for rows in (300, 40, 300):
        x = oracle.bf16_round(rng.standard_normal((rows, hidden)).astype(np.float32))
        res = oracle.bf16_round(rng.standard_normal((rows, hidden)).astype(np.float32))
        y = ffn.run(_dev(x, torch.bfloat16), _dev(res, torch.bfloat16))
        torch.cuda.synchronize()
        xp, xs, xr = oracle.quantize_nvfp4_rowscale(x)
        gate_up = oracle.matmul_nt(oracle.dequantize_tiled(xp, xs), oracle.dequantize_weight(gp, gs), alpha=float(gg), row_scale=xr)
        ap, as_ = oracle.silu_mul_halves_quantize_nvfp4(gate_up, in_scale)
        ref = oracle.matmul_nt(oracle.dequantize_tiled(ap, as_), oracle.dequantize_weight(dp, ds), alpha=float(dg) * in_scale) + res
        ok, stats = gemm_close(to_np(y), ref, rel=2e-2, abs_frac=2e-2)  # two quantized GEMMs in a row, bf16 output
        assert ok, stats
    assert sorted(ffn._plans) == [40, 300]  # one pair of plans per distinct row count, reused on the third call
