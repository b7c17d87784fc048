"""Helpers shared by the GPU parity tests."""
import numpy as np
import pytest


def require_cuda():
    torch = pytest.importorskip("torch")
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    return torch


def gemm_close(y, ref, rel=1e-2, abs_frac=1e-2):
    """|y - ref| <= max(tau_abs, rel * |ref|) with tau_abs = abs_frac * rms(ref): the reference's mixed
    criterion (crates/eider-cuda/src/cublaslt/fp4_tn.rs:1534) with the floor scaled to the data."""
    y = np.asarray(y, np.float64)
    ref = np.asarray(ref, np.float64)
    tau = abs_frac * float(np.sqrt(np.mean(ref * ref))) + 1e-30
    err = np.abs(y - ref)
    bound = np.maximum(tau, rel * np.abs(ref))
    bad = err > bound
    big = np.abs(ref) >= tau
    max_rel = float(np.max(err[big] / np.abs(ref[big]))) if big.any() else 0.0
    return (not bad.any()), {"max_abs_err": float(err.max()), "max_rel_err_over_floor": max_rel, "tau_abs": tau,
                             "bad": int(bad.sum()), "total": int(bad.size)}


def to_np(t):
    import torch
    if t.dtype == torch.bfloat16:
        return t.float().cpu().numpy()
    return t.cpu().numpy()
