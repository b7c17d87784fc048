"""numpy front-end of the CPU oracle (oracle/eider_oracle.c).

TEST INFRASTRUCTURE ONLY.  Importable from tests/, __graft_entry__.smoke() and the
cpu_baseline / reference legs of bench.py; the shipped package never imports it.

Parity status: pinned (see tests/test_oracle_golden.py for the reference's known-answer
vectors and tests/test_oracle_ref.py for the cross-check against the reference's own C++
conversion oracle compiled into oracle/_ref/).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_DIR = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_DIR, "liboracle.so")
_REF_PATH = os.path.join(_DIR, "_ref", "libfp4_oracle.so")


def build(ref: bool = True) -> None:
    """Compile liboracle.so and, when a checkout of the reference is found (REFERENCE_ROOT, or a `reference`
    directory beside the repository), its C++ conversion oracle into oracle/_ref."""
    subprocess.run(["make", "-C", _DIR, "all"], check=True, capture_output=True)
    ref_root = os.environ.get("REFERENCE_ROOT") or os.path.join(os.path.dirname(os.path.dirname(_DIR)), "reference")
    if ref and os.path.exists(os.path.join(ref_root, "crates/eider-cuda/native/fp4_oracle.cpp")):
        subprocess.run(["make", "-C", _DIR, "ref", f"REFERENCE_ROOT={ref_root}"], check=True,
                       capture_output=True)


def _load() -> C.CDLL:
    if not os.path.exists(_LIB_PATH):
        build(ref=False)
    return C.CDLL(_LIB_PATH)


_lib = _load()

_u8p = np.ctypeslib.ndpointer(np.uint8, flags="C_CONTIGUOUS")
_u16p = np.ctypeslib.ndpointer(np.uint16, flags="C_CONTIGUOUS")
_u32p = np.ctypeslib.ndpointer(np.uint32, flags="C_CONTIGUOUS")
_f32p = np.ctypeslib.ndpointer(np.float32, flags="C_CONTIGUOUS")
_sz = C.c_size_t


def _sig(name, res, *args):
    fn = getattr(_lib, name)
    fn.restype = res
    fn.argtypes = list(args)
    return fn


_e2m1_code = _sig("oracle_e2m1_code", C.c_uint8, C.c_float)
_e2m1_value = _sig("oracle_e2m1_value", C.c_float, C.c_uint8)
_e4m3_value = _sig("oracle_e4m3_value", C.c_float, C.c_uint8)
_e8m0_value = _sig("oracle_e8m0_value", C.c_float, C.c_uint8)
_ue4m3_code = _sig("oracle_ue4m3_code", C.c_uint8, C.c_float)
_e4m3_code = _sig("oracle_e4m3_code", C.c_uint8, C.c_float)
_layout_len = _sig("oracle_scale_layout_len", _sz, _sz, _sz)
_tiled_off = _sig("oracle_tiled_scale_offset", _sz, _sz, _sz, _sz)
_pack = _sig("oracle_pack_e2m1", None, _f32p, _sz, _u8p)
_to_tiled = _sig("oracle_scales_to_tiled", None, _u8p, _sz, _sz, _u8p)
_quant = _sig("oracle_quantize_nvfp4", None, _f32p, _sz, _sz, C.c_float, _u8p, _u8p)
_quant_row = _sig("oracle_quantize_nvfp4_rowscale", None, _f32p, _sz, _sz, _u8p, _u8p, _f32p)
_quant_w = _sig("oracle_quantize_weight", None, _f32p, _sz, _sz, C.c_float, _u8p, _u8p)
_w_global = _sig("oracle_weight_global_scale", C.c_float, _f32p, _sz)
_deq_rm = _sig("oracle_dequantize_rowmajor_scales", None, _u8p, _u8p, _sz, _sz, _f32p)
_deq_t = _sig("oracle_dequantize_tiled_scales", None, _u8p, _u8p, _sz, _sz, _f32p)
_matmul = _sig("oracle_matmul_nt", None, _f32p, _f32p, _sz, _sz, _sz, C.c_float, C.c_void_p,
               C.c_void_p, _f32p)
_linear_host = _sig("oracle_nvfp4_linear_host", None, _f32p, _sz, _u8p, _u8p, C.c_float, _sz, _sz,
                    _f32p, _f32p, C.c_int)
_max_threads = _sig("oracle_max_threads", C.c_int)
_set_threads = _sig("oracle_set_threads", None, C.c_int)
_q8_dyn = _sig("oracle_quantize_fp8_dynamic", None, _f32p, _sz, _sz, _u8p, _f32p)
_q8_static = _sig("oracle_quantize_fp8_static", None, _f32p, _sz, C.c_float, _u8p)
_q8_w = _sig("oracle_quantize_fp8_weight", None, _f32p, _sz, _sz, _u8p, _f32p)
_fp8_linear = _sig("oracle_fp8_linear", None, _u8p, _f32p, _u8p, _f32p, _sz, _sz, _sz, _f32p)
_topk = _sig("oracle_moe_topk", None, _f32p, _sz, _sz, _sz, C.c_int, _u32p, _f32p)
_sort = _sig("oracle_moe_sort_routes", None, _u32p, _sz, _sz, _u32p, _u32p, _u32p, _u32p, _u32p)
_scale_base = _sig("oracle_moe_scale_base", _sz, C.c_uint32, _u32p, _sz)
_gather_q = _sig("oracle_moe_gather_quantize", None, _f32p, _u32p, _u32p, _u32p, _sz, _sz, _sz, _sz,
                 C.c_int, _u8p, _u8p)
_silu_q = _sig("oracle_moe_silu_mul_quantize", None, _u16p, _u32p, _u32p, _sz, _sz, _sz, _u8p, _u8p,
               C.c_void_p)
_silu_dense = _sig("oracle_silu_mul_halves_quantize_nvfp4", None, _f32p, _sz, _sz, C.c_float, _u8p, _u8p, C.c_void_p)
_rms_q = _sig("oracle_rms_norm_quantize_nvfp4", None, _f32p, _f32p, _sz, _sz, C.c_float, C.c_float, _u8p, _u8p, C.c_void_p)
_rms_add_q = _sig("oracle_rms_norm_add_then_rms_norm_quantize_nvfp4", None, _f32p, _f32p, _f32p, _f32p, _f32p, _sz, _sz,
                  C.c_float, C.c_float, C.c_float, _u8p, _u8p, C.c_void_p)
_rms_pair = _sig("oracle_rms_norm_quantize_nvfp4_pair", None, _f32p, _f32p, _sz, _sz, C.c_float, C.c_float, _u8p, _u8p, _u8p, _u8p)
_grouped = _sig("oracle_moe_grouped_gemm", None, _u8p, _u8p, _u32p, _sz, _sz, _u8p, _u8p, _f32p, _sz,
                _sz, _u16p)
_combine = _sig("oracle_moe_combine", None, _u32p, _f32p, _u16p, _sz, _sz, _sz, _f32p)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


# ---- scalar codecs -------------------------------------------------------------------------
def e2m1_code(v: float) -> int:
    return int(_e2m1_code(float(v)))


def e2m1_value(c: int) -> float:
    return float(_e2m1_value(int(c)))


def e4m3_value(c: int) -> float:
    return float(_e4m3_value(int(c)))


def e8m0_value(c: int) -> float:
    return float(_e8m0_value(int(c)))


def ue4m3_code(v: float) -> int:
    return int(_ue4m3_code(float(v)))


def e4m3_code(v: float) -> int:
    return int(_e4m3_code(float(v)))


def pack_e2m1(values) -> np.ndarray:
    v = _f32(values)
    out = np.zeros((v.size + 1) // 2, np.uint8)
    _pack(v, v.size, out)
    return out


def scale_layout_len(outer: int, inner: int) -> int:
    return int(_layout_len(outer, inner))


def tiled_scale_offset(outer: int, block: int, inner: int) -> int:
    return int(_tiled_off(outer, block, inner))


def scales_to_tiled(row_major: np.ndarray, out_features: int, in_features: int) -> np.ndarray:
    src = np.ascontiguousarray(row_major, np.uint8).reshape(-1)
    out = np.zeros(scale_layout_len(out_features, in_features), np.uint8)
    _to_tiled(src, out_features, in_features, out)
    return out


def bf16_round(x: np.ndarray) -> np.ndarray:
    """f32 -> nearest-even bf16 -> f32 (crates/eider-cuda/src/format.rs:368-376)."""
    bits = _f32(x).view(np.uint32)
    lsb = (bits >> 16) & 1
    rounded = (bits + 0x7FFF + lsb) & 0xFFFF0000
    return rounded.astype(np.uint32).view(np.float32)


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    bits = _f32(x).view(np.uint32)
    lsb = (bits >> 16) & 1
    return ((bits + 0x7FFF + lsb) >> 16).astype(np.uint16)


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, np.uint16).astype(np.uint32) << 16).view(np.float32)


# ---- NVFP4 ---------------------------------------------------------------------------------
def quantize_nvfp4(x: np.ndarray, input_scale: float = 1.0):
    """[tokens, K] f32 -> (packed [tokens, K/2] u8, tiled scales u8)."""
    x = _f32(x)
    t, k = x.shape
    packed = np.zeros((t, k // 2), np.uint8)
    scales = np.zeros(scale_layout_len(t, k), np.uint8)
    _quant(x, t, k, float(input_scale), packed, scales)
    return packed, scales


def quantize_nvfp4_rowscale(x: np.ndarray):
    x = _f32(x)
    t, k = x.shape
    packed = np.zeros((t, k // 2), np.uint8)
    scales = np.zeros(scale_layout_len(t, k), np.uint8)
    row = np.zeros(t, np.float32)
    _quant_row(x, t, k, packed, scales, row)
    return packed, scales, row


def weight_global_scale(w: np.ndarray) -> float:
    w = _f32(w)
    return float(_w_global(w.reshape(-1), w.size))


def quantize_weight(w: np.ndarray, global_scale: float | None = None):
    """[N, K] f32 -> (packed [N, K/2], row-major scales [N, K/16], weight_scale_2)."""
    w = _f32(w)
    n, k = w.shape
    g = weight_global_scale(w) if global_scale is None else float(global_scale)
    packed = np.zeros((n, k // 2), np.uint8)
    scales = np.zeros((n, k // 16), np.uint8)
    _quant_w(w, n, k, g, packed, scales)
    return packed, scales, np.float32(g)


def dequantize_weight(packed: np.ndarray, scales_row_major: np.ndarray) -> np.ndarray:
    n, kh = packed.shape
    out = np.zeros((n, kh * 2), np.float32)
    _deq_rm(np.ascontiguousarray(packed), np.ascontiguousarray(scales_row_major).reshape(-1), n,
            kh * 2, out)
    return out


def dequantize_tiled(packed: np.ndarray, scales_tiled: np.ndarray) -> np.ndarray:
    t, kh = packed.shape
    out = np.zeros((t, kh * 2), np.float32)
    _deq_t(np.ascontiguousarray(packed), np.ascontiguousarray(scales_tiled), t, kh * 2, out)
    return out


def matmul_nt(a: np.ndarray, w: np.ndarray, alpha: float = 1.0, row_scale=None, col_scale=None):
    a, w = _f32(a), _f32(w)
    m, k = a.shape
    n = w.shape[0]
    y = np.zeros((m, n), np.float32)
    rs = _f32(row_scale) if row_scale is not None else None
    cs = _f32(col_scale) if col_scale is not None else None
    _matmul(a, w, m, n, k, float(alpha), rs.ctypes.data if rs is not None else None,
            cs.ctypes.data if cs is not None else None, y)
    return y


def nvfp4_linear_host(x: np.ndarray, packed: np.ndarray, scales_row_major: np.ndarray,
                      weight_scale_2: float, threads: int = 0, scratch: np.ndarray | None = None):
    """The reference's host path: unpack to f32, then the f32 triple loop."""
    x = _f32(x)
    m, k = x.shape
    n = packed.shape[0]
    if scratch is None:
        scratch = np.empty(n * k, np.float32)
    y = np.zeros((m, n), np.float32)
    _linear_host(x, m, np.ascontiguousarray(packed), np.ascontiguousarray(scales_row_major).reshape(-1),
                 float(weight_scale_2), n, k, scratch, y, int(threads))
    return y


def max_threads() -> int:
    return int(_max_threads())


def set_threads(n: int) -> None:
    _set_threads(int(n))


# ---- FP8 -----------------------------------------------------------------------------------
def quantize_fp8_dynamic(x: np.ndarray):
    x = _f32(x)
    r, c = x.shape
    q = np.zeros((r, c), np.uint8)
    s = np.zeros(r, np.float32)
    _q8_dyn(x, r, c, q, s)
    return q, s


def quantize_fp8_static(x: np.ndarray, input_scale: float):
    x = _f32(x)
    q = np.zeros(x.shape, np.uint8)
    _q8_static(x.reshape(-1), x.size, float(input_scale), q.reshape(-1))
    return q


def quantize_fp8_weight(w: np.ndarray):
    w = _f32(w)
    n, k = w.shape
    q = np.zeros((n, k), np.uint8)
    s = np.zeros(n, np.float32)
    _q8_w(w, n, k, q, s)
    return q, s


def fp8_linear(xq, s_x, wq, s_w):
    xq = np.ascontiguousarray(xq, np.uint8)
    wq = np.ascontiguousarray(wq, np.uint8)
    m, k = xq.shape
    n = wq.shape[0]
    y = np.zeros((m, n), np.float32)
    _fp8_linear(xq, _f32(s_x), wq, _f32(s_w), m, n, k, y)
    return y


def e4m3_decode(codes: np.ndarray) -> np.ndarray:
    lut = np.array([e4m3_value(i) for i in range(256)], np.float32)
    return lut[np.asarray(codes, np.uint8)]


# ---- MoE -----------------------------------------------------------------------------------
def moe_topk(logits: np.ndarray, k: int, norm_topk_prob: bool):
    lg = _f32(logits)
    t, e = lg.shape
    idx = np.zeros((t, k), np.uint32)
    w = np.zeros((t, k), np.float32)
    _topk(lg, t, e, k, int(bool(norm_topk_prob)), idx, w)
    return idx, w


def moe_sort_routes(indices: np.ndarray, experts: int):
    ind = np.ascontiguousarray(indices, np.uint32).reshape(-1)
    r = ind.size
    counts = np.zeros(experts, np.uint32)
    offsets = np.zeros(experts + 1, np.uint32)
    sorted_routes = np.zeros(r, np.uint32)
    sorted_experts = np.zeros(r, np.uint32)
    inverse = np.zeros(r, np.uint32)
    _sort(ind, r, experts, counts, offsets, sorted_routes, sorted_experts, inverse)
    return counts, offsets, sorted_routes, sorted_experts, inverse


def moe_scale_tile_bytes(k: int) -> int:
    """Bytes of one 128-row scale tile row-block: 128 * padded K/16."""
    return 128 * ((k // 16 + 3) // 4 * 4)


def moe_scale_bytes(routes: int, experts: int, k: int) -> int:
    """Upper bound used by the reference: (ceil(routes/128) + experts) tiles."""
    return ((routes + 127) // 128 + experts) * moe_scale_tile_bytes(k)


def moe_scale_base(expert: int, offsets: np.ndarray, tile_bytes: int) -> int:
    return int(_scale_base(expert, np.ascontiguousarray(offsets, np.uint32), tile_bytes))


def moe_gather_quantize(x, sorted_routes, sorted_experts, offsets, routes_per_row, experts,
                        gather_rows=True):
    x = _f32(x)
    k = x.shape[1]
    r = sorted_routes.size
    tile = moe_scale_tile_bytes(k)
    packed = np.zeros((r, k // 2), np.uint8)
    scales = np.zeros(moe_scale_bytes(r, experts, k), np.uint8)
    _gather_q(x, sorted_routes, sorted_experts, offsets, r, routes_per_row, k, tile,
              int(gather_rows), packed, scales)
    return packed, scales


def moe_silu_mul_quantize(gate_up_bits, sorted_experts, offsets, experts, want_act=False):
    gu = np.ascontiguousarray(gate_up_bits, np.uint16)
    r, two_k = gu.shape
    k = two_k // 2
    tile = moe_scale_tile_bytes(k)
    packed = np.zeros((r, k // 2), np.uint8)
    scales = np.zeros(moe_scale_bytes(r, experts, k), np.uint8)
    act = np.zeros((r, k), np.float32) if want_act else None
    _silu_q(gu, sorted_experts, offsets, r, k, tile, packed, scales,
            act.ctypes.data if act is not None else None)
    return (packed, scales, act) if want_act else (packed, scales)


def silu_mul_halves_quantize_nvfp4(gate_up, input_scale=1.0, want_act=False):
    """gate_up [tokens, 2K] f32 -> (packed [tokens, K/2], tiled scales[, fp32 products]); non_gemm.cu:559-629."""
    gu = _f32(gate_up)
    if gu.ndim == 1:
        gu = gu[None]
    t, two_k = gu.shape
    k = two_k // 2
    packed = np.zeros((t, k // 2), np.uint8)
    scales = np.zeros(scale_layout_len(t, k), np.uint8)
    act = np.zeros((t, k), np.float32) if want_act else None
    _silu_dense(np.ascontiguousarray(gu), t, k, float(input_scale), packed, scales, act.ctypes.data if act is not None else None)
    return (packed, scales, act) if want_act else (packed, scales)


def rms_norm_quantize_nvfp4(x, weight, eps=1e-6, input_scale=1.0, want_norm=False):
    """x [rows, cols] f32, weight [cols] -> (packed, tiled scales[, normalised fp32 values]); non_gemm.cu:193-288."""
    x = _f32(x)
    rows, cols = x.shape
    packed = np.zeros((rows, (cols + 1) // 2), np.uint8)
    scales = np.zeros(scale_layout_len(rows, cols), np.uint8)
    norm = np.zeros((rows, cols), np.float32) if want_norm else None
    _rms_q(np.ascontiguousarray(x), _f32(weight), rows, cols, float(eps), float(input_scale), packed, scales,
           norm.ctypes.data if norm is not None else None)
    return (packed, scales, norm) if want_norm else (packed, scales)


def rms_norm_quantize_nvfp4_pair(x, weight, eps=1e-6, input_scale=1.0):
    """non_gemm.cu:290-419 -> (packed, scales, residual_packed, residual_scales)."""
    x = _f32(x)
    rows, cols = x.shape
    packed = np.zeros((rows, cols // 2), np.uint8)
    rpacked = np.zeros((rows, cols // 2), np.uint8)
    scales = np.zeros(scale_layout_len(rows, cols), np.uint8)
    rscales = np.zeros(scale_layout_len(rows, cols), np.uint8)
    _rms_pair(np.ascontiguousarray(x), _f32(weight), rows, cols, float(eps), float(input_scale), packed, scales, rpacked, rscales)
    return packed, scales, rpacked, rscales


def rms_norm_add_then_rms_norm_quantize_nvfp4(x, input_weight, residual, quant_weight, input_eps=1e-6, quant_eps=1e-6,
                                              input_scale=1.0):
    """non_gemm.cu:746-870 -> (h [rows, cols] f32, packed, tiled scales, normalised fp32 values of the second norm)."""
    x = _f32(x)
    rows, cols = x.shape
    h = np.zeros((rows, cols), np.float32)
    packed = np.zeros((rows, cols // 2), np.uint8)
    scales = np.zeros(scale_layout_len(rows, cols), np.uint8)
    norm = np.zeros((rows, cols), np.float32)
    _rms_add_q(np.ascontiguousarray(x), _f32(input_weight), np.ascontiguousarray(_f32(residual)), h, _f32(quant_weight), rows, cols,
               float(input_eps), float(quant_eps), float(input_scale), packed, scales, norm.ctypes.data)
    return h, packed, scales, norm


def moe_grouped_gemm(act_packed, act_scales, offsets, w_packed, w_scales, alpha):
    """w_packed [E, N, K/2], w_scales [E, N, K/16], alpha [E] -> bf16 bits [routes, N]."""
    e, n, kh = w_packed.shape
    k = kh * 2
    r = act_packed.shape[0]
    out = np.zeros((r, n), np.uint16)
    _grouped(np.ascontiguousarray(act_packed), np.ascontiguousarray(act_scales),
             np.ascontiguousarray(offsets, np.uint32), e, moe_scale_tile_bytes(k),
             np.ascontiguousarray(w_packed).reshape(-1), np.ascontiguousarray(w_scales).reshape(-1),
             _f32(alpha), n, k, out)
    return out


def moe_combine(route_to_sorted, route_weights, sorted_bf16_bits, rows, routes_per_row):
    src = np.ascontiguousarray(sorted_bf16_bits, np.uint16)
    ln = src.shape[1]
    out = np.zeros((rows, ln), np.float32)
    _combine(np.ascontiguousarray(route_to_sorted, np.uint32).reshape(-1),
             _f32(route_weights).reshape(-1), src, rows, ln, routes_per_row, out)
    return out


def gelu_tanh_mul(gate: np.ndarray, up: np.ndarray) -> np.ndarray:
    """0.5 g (1 + tanh(sqrt(2/pi) (g + 0.044715 g^3))) * up in f32, operation by operation
    (crates/eider-cuda/native/non_gemm.cu:446-451); tanh is numpy's, so the last place may differ from the device's."""
    g, u = _f32(gate), _f32(up)
    cubic = (g * g) * g
    inner = np.float32(0.7978845608028654) * (g + np.float32(0.044715) * cubic)
    return ((np.float32(0.5) * g) * (np.float32(1.0) + np.tanh(inner).astype(np.float32))) * u


def quantize_nvfp4_vector_simple_scales(x: np.ndarray, input_scale: float = 1.0):
    """One vector, one scale byte per 16 values in plain order (crates/eider-cuda/native/non_gemm.cu:510-541):
    -> (packed [(n + 1) // 2], scales [ceil(n / 16)])."""
    v = _f32(x).reshape(-1)
    n = v.size
    blocks = (n + 15) // 16
    padded = np.zeros((1, blocks * 16), np.float32)
    padded[0, :n] = v
    packed, tiled = quantize_nvfp4(padded, input_scale)
    scales = np.array([tiled[tiled_scale_offset(0, b, blocks * 16)] for b in range(blocks)], np.uint8)
    return packed.reshape(-1)[:(n + 1) // 2].copy(), scales


def moe_quantize_rows_into_expert_tiles(values: np.ndarray, sorted_experts, offsets, experts: int):
    """Quantize already sorted f32 rows (unit global scale) into expert-major NVFP4 rows and per-expert scale tiles
    (crates/eider-cuda/native/non_gemm.cu:2554-2557, 2621-2676): -> (packed [R, K/2], scales)."""
    v = _f32(values)
    r, k = v.shape
    return moe_gather_quantize(v, np.arange(r, dtype=np.uint32), np.ascontiguousarray(sorted_experts, np.uint32),
                               np.ascontiguousarray(offsets, np.uint32), 1, experts, gather_rows=False)


def moe_calibrated_values(x: np.ndarray, input_scales, sorted_routes, sorted_experts, routes_per_row: int,
                          relu_squared: bool = False) -> np.ndarray:
    """The f32 values the per-expert calibrated quantizer sees (crates/eider-cuda/native/non_gemm.cu:2562-2585):
    value = x * (1 / input_scales[expert]); relu_squared: x = max(bf16 row, 0)^2 of the sorted row itself."""
    inv = (np.float32(1.0) / _f32(input_scales))[np.asarray(sorted_experts, np.int64)][:, None]
    if relu_squared:
        v = np.maximum(_f32(x), np.float32(0.0))
        return (v * v) * inv
    rows = np.asarray(sorted_routes, np.int64) // routes_per_row
    return _f32(x)[rows] * inv


# ---- reference's own conversion oracle (oracle/_ref) ---------------------------------------
def load_reference_codec():
    """ctypes handle on oracle/_ref/libfp4_oracle.so or None when it was not built."""
    if not os.path.exists(_REF_PATH):
        return None
    lib = C.CDLL(_REF_PATH)
    lib.infer_cuda_e2m1_rn.restype = C.c_uint8
    lib.infer_cuda_e2m1_rn.argtypes = [C.c_float]
    lib.infer_cuda_e4m3_satfinite.restype = C.c_uint8
    lib.infer_cuda_e4m3_satfinite.argtypes = [C.c_float]
    return lib
