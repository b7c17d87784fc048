"""CUDA-core decode kernels against the oracle's dequantize + f32 dot (the reference's host path)."""
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


@pytest.mark.parametrize("batch,n,k", [(1, 64, 64), (1, 1000, 2048), (3, 136, 5120), (8, 256, 1040), (1, 13824, 5120)])
@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_w4a16_matvec(ops, oracle, batch, n, k, dtype):
    import torch
    rng = np.random.default_rng(n + k + batch)
    w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    packed, scales, g = oracle.quantize_weight(w)
    x = oracle.bf16_round(rng.standard_normal((batch, k)).astype(np.float32))
    wd = ops.ModelOptWeight.from_checkpoint(_dev(packed), _dev(scales), float(g))
    y = ops.nvfp4_w4a16_matvec(_dev(x, torch.bfloat16 if dtype == "bf16" else None), wd)
    ref = oracle.nvfp4_linear_host(x, packed, scales, float(g))
    ok, stats = gemm_close(to_np(y), ref, rel=1e-2 if dtype == "bf16" else 1e-4, abs_frac=1e-2 if dtype == "bf16" else 1e-4)
    assert ok, stats


def test_w4a16_rejects_bad_arguments(ops):
    from eider_b200 import _lib
    lib = _lib.load()
    assert lib.infer_nvfp4_w4a16_matvec_f32_on_stream(None, None, None, None, 16, 16, 1.0, None) == 1
    import torch
    t = torch.zeros(64, device="cuda")
    assert lib.infer_nvfp4_w4a16_matvec_f32_on_stream(t.data_ptr(), t.data_ptr(), t.data_ptr(), t.data_ptr(), 4, 24, 1.0, None) == 1


@pytest.mark.parametrize("m,n,k", [(1, 128, 256), (4, 200, 5120), (7, 96, 1000)])
def test_fp8_prequantized_simt(ops, oracle, m, n, k):
    rng = np.random.default_rng(m + n + k)
    w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    wq, ws = oracle.quantize_fp8_weight(w)
    x = rng.standard_normal((m, k)).astype(np.float32)
    xq, xs = oracle.quantize_fp8_dynamic(x)
    y = ops.fp8_linear_prequantized_simt(_dev(xq), _dev(xs), _dev(wq), _dev(ws))
    ref = oracle.fp8_linear(xq, xs, wq, ws)
    ok, stats = gemm_close(to_np(y), ref, rel=1e-4, abs_frac=1e-4)
    assert ok, stats
