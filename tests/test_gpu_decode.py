"""Tensor-core decode path (1..64 tokens): NVFP4 W4A16 through the residual activation expansion and FP8 W8A8,
against the oracle's host path (unpack + f32 dot, the reference's own CPU form)."""
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


@pytest.mark.parametrize("terms", [1, 4, 8])
def test_expansion_reconstructs_activation(ops, oracle, terms):
    rng = np.random.default_rng(terms)
    x = rng.standard_normal((3, 2048)).astype(np.float32) * np.exp(rng.uniform(-4, 4, (3, 2048))).astype(np.float32)
    packed, scales, col = ops.expand_nvfp4_terms(_dev(x), terms)
    deq = oracle.dequantize_tiled(packed.cpu().numpy(), scales.cpu().numpy()) * col.cpu().numpy()[:, None]
    rec = deq.reshape(3, terms, -1).sum(axis=1)
    amax = np.abs(x).max(axis=1, keepdims=True)
    bound = {1: 0.2, 4: 2e-3, 8: 2e-5}[terms]
    assert np.all(np.abs(rec - x) <= bound * amax)
    if terms == 1:  # term 0 is exactly the row-scale quantizer
        p0, s0, r0 = oracle.quantize_nvfp4_rowscale(x)
        assert np.array_equal(packed.cpu().numpy(), p0)
        assert np.array_equal(col.cpu().numpy(), r0)


@pytest.mark.parametrize("tokens,n,k", [(1, 128, 256), (1, 13824, 5120), (1, 5120, 13824), (2, 640, 1056), (3, 1000, 2048),
                                        (4, 5120, 13824), (8, 7168, 5120),
                                        (32, 520, 1024), (33, 512, 1024), (64, 2048, 5120)])
@pytest.mark.parametrize("dtype", ["bf16", "f32"])
def test_nvfp4_w4a16_decode(ops, oracle, tokens, n, k, dtype):
    import torch
    rng = np.random.default_rng(tokens + n + k)
    w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    packed, scales, g = oracle.quantize_weight(w)
    x = rng.standard_normal((tokens, k)).astype(np.float32)
    if dtype == "bf16":
        x = oracle.bf16_round(x)
    wd = ops.ModelOptWeight.from_checkpoint(_dev(packed), _dev(scales), float(g))
    plan = ops.Nvfp4DecodePlan(64 if tokens > 32 else 32 if tokens > 1 else 1, n, k)
    y = plan.run(_dev(x, torch.bfloat16 if dtype == "bf16" else None), wd, out_dtype=torch.float32)
    y2 = plan.run(_dev(x, torch.bfloat16 if dtype == "bf16" else None), wd, out_dtype=torch.float32)  # counters self-reset
    torch.cuda.synchronize()
    assert plan.status() == 0
    ref = oracle.nvfp4_linear_host(x, packed, scales, float(g))
    # eight residual terms carry the activation essentially exactly; four terms keep ~1e-3 of the block maximum
    # and that is also what the single-launch path uses for one or two bf16 tokens (bf16 itself resolves 4e-3)
    tol = 1e-4 if tokens <= 32 else 1e-2
    if dtype == "bf16":
        tol = max(tol, 2e-3)  # bf16 activations always take four terms
    ok, stats = gemm_close(to_np(y), ref, rel=tol, abs_frac=tol)
    assert ok, stats
    assert torch.equal(y, y2)


@pytest.mark.parametrize("tokens,n,k", [(1, 128, 256), (1, 13824, 5120), (1, 5120, 13824), (2, 640, 1056), (3, 1000, 2048),
                                        (4, 1024, 2080), (5, 5120, 13824), (8, 13824, 5120)])
@pytest.mark.parametrize("dtype", ["bf16", "f32"])
def test_nvfp4_w4a16_decode_on_prepared_operand(ops, oracle, tokens, n, k, dtype):
    # the producer of x expands it once (operand object); the GEMV copies its slice instead of expanding it itself
    import torch
    if dtype == "f32" and tokens > 4:
        pytest.skip("eight terms x more than four tokens do not fit the 32 operand rows")
    rng = np.random.default_rng(tokens * 3 + n + k)
    w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    packed, scales, g = oracle.quantize_weight(w)
    x = rng.standard_normal((tokens, k)).astype(np.float32)
    if dtype == "bf16":
        x = oracle.bf16_round(x)
    wd = ops.ModelOptWeight.from_checkpoint(_dev(packed), _dev(scales), float(g))
    plan = ops.Nvfp4DecodePlan(8, n, k)
    operand = ops.Nvfp4DecodeOperand(8, k)
    xd = _dev(x, torch.bfloat16 if dtype == "bf16" else None)
    y = plan.run_prepared(operand.expand(xd), wd, out_dtype=torch.float32)
    y2 = plan.run_prepared(operand, wd, out_dtype=torch.float32)  # the operand serves several GEMVs; counters self-reset
    torch.cuda.synchronize()
    assert plan.status() == 0
    ref = oracle.nvfp4_linear_host(x, packed, scales, float(g))
    tol = 2e-3 if dtype == "bf16" else 1e-4
    ok, stats = gemm_close(to_np(y), ref, rel=tol, abs_frac=tol)
    assert ok, stats
    assert torch.equal(y, y2)
    # a smaller batch through the same operand afterwards (rows of the earlier, larger batch are left behind it)
    if tokens > 1:
        y1 = plan.run_prepared(operand.expand(xd[:1].contiguous()), wd, out_dtype=torch.float32)
        torch.cuda.synchronize()
        ok, stats = gemm_close(to_np(y1), ref[:1], rel=tol, abs_frac=tol)
        assert ok, stats


def test_nvfp4_decode_terms_follow_the_call_not_the_plan(ops, oracle):
    # a plan made for 64 tokens still gives f32 activations eight residual terms when the call's tokens fit
    import torch
    rng = np.random.default_rng(21)
    n, k = 1024, 2048
    w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    packed, scales, g = oracle.quantize_weight(w)
    wd = ops.ModelOptWeight.from_checkpoint(_dev(packed), _dev(scales), float(g))
    plan = ops.Nvfp4DecodePlan(64, n, k)
    for tokens, tol in ((8, 1e-4), (32, 1e-4), (33, 1e-2)):
        x = rng.standard_normal((tokens, k)).astype(np.float32)
        y = plan.run(_dev(x), wd, out_dtype=torch.float32)
        torch.cuda.synchronize()
        assert plan.status() == 0
        ok, stats = gemm_close(to_np(y), oracle.nvfp4_linear_host(x, packed, scales, float(g)), rel=tol, abs_frac=tol)
        assert ok, (tokens, stats)


def test_nvfp4_decode_bf16_out_and_beta(ops, oracle):
    import torch
    rng = np.random.default_rng(9)
    n, k = 640, 1024
    w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    packed, scales, g = oracle.quantize_weight(w)
    x = oracle.bf16_round(rng.standard_normal((2, k)).astype(np.float32))
    wd = ops.ModelOptWeight.from_checkpoint(_dev(packed), _dev(scales), float(g))
    plan = ops.Nvfp4DecodePlan(2, n, k)
    ref = oracle.nvfp4_linear_host(x, packed, scales, float(g))
    y = plan.run(_dev(x, torch.bfloat16), wd)
    ok, stats = gemm_close(to_np(y), ref)
    assert ok, stats
    res = rng.standard_normal((2, n)).astype(np.float32)
    out = _dev(res)
    plan.run(_dev(x, torch.bfloat16), wd, out=out, beta=1.0)  # residual add fused, as LinearDecodeOp does with beta = 1
    ok, stats = gemm_close(to_np(out), ref + res, rel=2e-3, abs_frac=2e-3)  # bf16 input: four residual terms
    assert ok, stats


@pytest.mark.parametrize("tokens", [1, 8, 32, 64])
def test_fp8_decode_qkv(ops, oracle, tokens):
    # FP8 attention projection: K = 5120, N = 7168 (fused QKV), per-channel weight scales, per-token activations
    import torch
    n, k = 7168, 5120
    rng = np.random.default_rng(tokens)
    w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    x = oracle.bf16_round(rng.standard_normal((tokens, k)).astype(np.float32))
    wq, ws = oracle.quantize_fp8_weight(w)
    xq, xs = oracle.quantize_fp8_dynamic(x)
    plan = ops.Fp8DecodePlan(64, n, k)
    y = plan.run(_dev(x, torch.bfloat16), _dev(wq), _dev(ws))
    torch.cuda.synchronize()
    assert plan.status() == 0
    ref = oracle.fp8_linear(xq, xs, wq, ws)
    ok, stats = gemm_close(to_np(y), ref)
    assert ok, stats


@pytest.mark.parametrize("tokens,n,k", [(1, 7168, 5120), (5, 7168, 5120), (16, 1000, 528), (17, 7168, 5120), (33, 640, 2064), (64, 7168, 5120)])
def test_fp8_decode_on_quantized_activations(ops, oracle, tokens, n, k):
    # the producer of x runs the per-token quantizer; the GEMV takes its codes and scales (and equals the call that
    # quantizes for itself, bit for bit, wherever that call takes the same route)
    import torch
    rng = np.random.default_rng(tokens * 5 + n)
    w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    x = oracle.bf16_round(rng.standard_normal((tokens, k)).astype(np.float32))
    wq, ws = oracle.quantize_fp8_weight(w)
    xq_ref, xs_ref = oracle.quantize_fp8_dynamic(x)
    xd = _dev(x, torch.bfloat16)
    xq, xs = ops.quantize_fp8_dynamic(xd)
    assert np.array_equal(to_np(xq), xq_ref) and np.array_equal(to_np(xs), xs_ref)
    wqd, wsd = _dev(wq), _dev(ws)
    plan = ops.Fp8DecodePlan(64, n, k)
    y = plan.run_quantized(xq, xs, wqd, wsd, out_dtype=torch.float32)
    y2 = plan.run_quantized(xq, xs, wqd, wsd, out_dtype=torch.float32)
    torch.cuda.synchronize()
    assert plan.status() == 0
    ok, stats = gemm_close(to_np(y), oracle.fp8_linear(xq_ref, xs_ref, wq, ws), rel=1e-4, abs_frac=1e-4)
    assert ok, stats
    assert torch.equal(y, y2)
    if tokens > 4:
        y3 = plan.run(xd, wqd, wsd, out_dtype=torch.float32)
        torch.cuda.synchronize()
        assert torch.equal(y, y3)


def test_fp8_decode_small_and_scalar_scale(ops, oracle):
    import torch
    n, k = 200, 528
    rng = np.random.default_rng(4)
    wq = rng.integers(0, 0x7E, (n, k)).astype(np.uint8) | (rng.integers(0, 2, (n, k)).astype(np.uint8) << 7)
    x = rng.standard_normal((5, k)).astype(np.float32)
    xq, xs = oracle.quantize_fp8_dynamic(x)
    plan = ops.Fp8DecodePlan(8, n, k)
    y = plan.run(_dev(x), _dev(wq), None, weight_scale=0.03125, out_dtype=torch.float32)
    ref = oracle.fp8_linear(xq, xs, wq, np.full(n, 0.03125, np.float32))
    ok, stats = gemm_close(to_np(y), ref, rel=1e-4, abs_frac=1e-4)
    assert ok, stats


@pytest.mark.parametrize("tokens", [1, 2, 3, 4, 7, 8])
@pytest.mark.parametrize("n,k", [(200, 528), (1000, 2048), (5120, 13824)])
def test_fp8_decode_single_launch(ops, oracle, tokens, n, k):
    # one to four tokens take the single-launch kernel (more go through the quantize kernel + GEMV pair) (quantizer inside the GEMV CTAs, K splits met in scratch):
    # same codes and scales as the stand-alone quantizer, partial row tiles, a K that is not a multiple of the stage
    import torch
    rng = np.random.default_rng(tokens * 31 + n)
    wq = rng.integers(0, 0x7E, (n, k)).astype(np.uint8) | (rng.integers(0, 2, (n, k)).astype(np.uint8) << 7)
    ws = (rng.uniform(0.5, 2.0, n) * 0.01).astype(np.float32)
    x = rng.standard_normal((tokens, k)).astype(np.float32) * np.exp(rng.uniform(-2, 2, (tokens, 1))).astype(np.float32)
    xq, xs = oracle.quantize_fp8_dynamic(x)
    plan = ops.Fp8DecodePlan(8, n, k)
    y = plan.run(_dev(x), _dev(wq), _dev(ws), out_dtype=torch.float32)
    y2 = plan.run(_dev(x), _dev(wq), _dev(ws), out_dtype=torch.float32)  # counters self-reset, fixed summation order
    torch.cuda.synchronize()
    assert plan.status() == 0
    ref = oracle.fp8_linear(xq, xs, wq, ws)
    ok, stats = gemm_close(to_np(y), ref, rel=1e-4, abs_frac=1e-4)
    assert ok, stats
    assert torch.equal(y, y2)


def test_decode_rejects_bad_arguments(ops):
    from eider_b200 import _lib
    lib = _lib.load()
    assert not lib.eider_b200_nvfp4_decode_create(65, 128, 128)
    assert not lib.eider_b200_nvfp4_decode_create(1, 128, 48)
    with pytest.raises(ops.ShapeError):
        ops.Nvfp4DecodePlan(0, 128, 128)
    plan = lib.eider_b200_nvfp4_decode_create(4, 128, 128)
    assert lib.eider_b200_nvfp4_w4a16_gemv_on_stream(plan, None, 1, 1, None, None, 1.0, None, None, 0.0, 1, None) == 1
    lib.eider_b200_decode_destroy(plan)


def test_prepared_activation_entry_points_reject_bad_arguments(ops):
    # argument checks of the operand object and of the GEMVs on prepared activations, all before any launch
    import torch
    from eider_b200 import _lib
    lib = _lib.load()
    assert not lib.eider_b200_nvfp4_decode_operand_create(9, 256)   # at most eight tokens
    assert not lib.eider_b200_nvfp4_decode_operand_create(1, 48)    # K in multiples of 32
    op = lib.eider_b200_nvfp4_decode_operand_create(8, 256)
    plan = lib.eider_b200_nvfp4_decode_create(8, 128, 256)
    other = lib.eider_b200_nvfp4_decode_create(8, 128, 512)
    assert op and plan and other
    x = torch.randn(8, 256, device="cuda")
    w = torch.zeros(128, 128, dtype=torch.uint8, device="cuda")
    s = torch.zeros(128 * 16, dtype=torch.uint8, device="cuda")
    y = torch.zeros(8, 128, dtype=torch.bfloat16, device="cuda")
    try:
        # nothing expanded yet: the operand holds no tokens
        assert lib.eider_b200_nvfp4_w4a16_gemv_prepared_on_stream(plan, op, w.data_ptr(), s.data_ptr(), 1.0, None, y.data_ptr(), 0.0, 1, None) == 1
        # eight terms x five f32 tokens do not fit the 32 operand rows; nine tokens exceed the operand
        assert lib.eider_b200_nvfp4_decode_operand_expand_on_stream(op, x.data_ptr(), 0, 5, None) == 1
        assert lib.eider_b200_nvfp4_decode_operand_expand_on_stream(op, x.data_ptr(), 1, 9, None) == 1
        assert lib.eider_b200_nvfp4_decode_operand_expand_on_stream(op, None, 1, 1, None) == 1
        assert lib.eider_b200_nvfp4_decode_operand_expand_on_stream(op, x.data_ptr(), 0, 4, None) == 0
        # a plan of another K, a missing weight, beta without C
        assert lib.eider_b200_nvfp4_w4a16_gemv_prepared_on_stream(other, op, w.data_ptr(), s.data_ptr(), 1.0, None, y.data_ptr(), 0.0, 1, None) == 1
        assert lib.eider_b200_nvfp4_w4a16_gemv_prepared_on_stream(plan, op, None, s.data_ptr(), 1.0, None, y.data_ptr(), 0.0, 1, None) == 1
        assert lib.eider_b200_nvfp4_w4a16_gemv_prepared_on_stream(plan, op, w.data_ptr(), s.data_ptr(), 1.0, None, y.data_ptr(), 0.5, 1, None) == 1
        assert lib.eider_b200_nvfp4_w4a16_gemv_prepared_on_stream(plan, op, w.data_ptr(), s.data_ptr(), 1.0, None, y.data_ptr(), 0.0, 1, None) == 0
        torch.cuda.synchronize()
        fplan = lib.eider_b200_fp8_decode_create(64, 128, 256)
        codes = torch.zeros(8, 256, dtype=torch.uint8, device="cuda")
        scales = torch.ones(8, device="cuda")
        w8 = torch.zeros(128, 256, dtype=torch.uint8, device="cuda")
        assert lib.eider_b200_fp8_linear_decode_quantized_on_stream(fplan, None, scales.data_ptr(), 8, w8.data_ptr(), None, 1.0, y.data_ptr(), 1, None) == 1
        assert lib.eider_b200_fp8_linear_decode_quantized_on_stream(fplan, codes.data_ptr(), None, 8, w8.data_ptr(), None, 1.0, y.data_ptr(), 1, None) == 1
        assert lib.eider_b200_fp8_linear_decode_quantized_on_stream(fplan, codes.data_ptr(), scales.data_ptr(), 65, w8.data_ptr(), None, 1.0, y.data_ptr(), 1, None) == 1
        assert lib.eider_b200_fp8_linear_decode_quantized_on_stream(plan, codes.data_ptr(), scales.data_ptr(), 8, w8.data_ptr(), None, 1.0, y.data_ptr(), 1, None) == 1
        assert lib.eider_b200_fp8_linear_decode_quantized_on_stream(fplan, codes.data_ptr(), scales.data_ptr(), 8, w8.data_ptr(), None, 1.0, y.data_ptr(), 1, None) == 0
        torch.cuda.synchronize()
        assert torch.all(y == 0)
        lib.eider_b200_decode_destroy(fplan)
    finally:
        lib.eider_b200_decode_destroy(plan)
        lib.eider_b200_decode_destroy(other)
        lib.eider_b200_nvfp4_decode_operand_destroy(op)
