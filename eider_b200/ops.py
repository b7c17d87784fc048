"""Host-side mirror of the reference's safe operator API for the quantized-linear path.

Names follow crates/eider-cuda (Nvfp4Matrix, ModelOptCublasLtWeight -> ModelOptWeight,
Fp4TnMatmulPlan, Fp8TnMatmulPlan, MoeSortedRoutes ...) so tests read like the reference's.  PyTorch
only owns device memory and streams here; every computation goes through the C ABI in
include/eider_b200.h.  Shape / format errors are raised on the host before any launch, as the
reference's wrappers do (crates/eider-cuda/src/kernels/non_gemm.rs:5672-5703).
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import torch

from . import _lib
from ._lib import check


class ShapeError(ValueError):
    """crates/eider-cuda/src/error.rs Error::Shape."""


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def _need(t: torch.Tensor, dtype, label: str) -> None:
    if not t.is_cuda or not t.is_contiguous() or t.dtype != dtype:
        raise ShapeError(f"{label}: expected contiguous CUDA tensor of {dtype}, got {t.dtype} cuda={t.is_cuda}")


def scale_layout_len(outer: int, inner: int) -> int:
    """ue4m3_scale_layout_len (crates/eider-cuda/src/format.rs:194-198)."""
    return int(_lib.load().eider_b200_nvfp4_scale_layout_len(outer, inner))


@dataclass
class Nvfp4Matrix:
    """Device NVFP4 matrix: packed E2M1 [rows, K/2] + tiled UE4M3 scales (crates/eider-cuda/src/matrix.rs:43-331)."""
    packed: torch.Tensor
    scales: torch.Tensor
    rows: int
    k: int
    row_scales: torch.Tensor | None = None  # per-row global scale when quantized on the fly

    @staticmethod
    def zeros(rows: int, k: int, device="cuda", row_scales: bool = False) -> "Nvfp4Matrix":
        if k % 16 != 0:
            raise ShapeError(f"NVFP4 needs K % 16 == 0, got {k}")
        return Nvfp4Matrix(
            torch.zeros(rows, k // 2, dtype=torch.uint8, device=device),
            torch.zeros(scale_layout_len(rows, k), dtype=torch.uint8, device=device),
            rows, k,
            torch.zeros(rows, dtype=torch.float32, device=device) if row_scales else None)


# ---- NVFP4 activation quantize ------------------------------------------------------------------
def quantize_nvfp4(x: torch.Tensor, input_scale: float = 1.0, out: Nvfp4Matrix | None = None) -> Nvfp4Matrix:
    """infer_quantize_nvfp4_col_major_f32_on_stream for x [tokens, K] (f32 or bf16), static scale."""
    lib = _lib.load()
    tokens, k = x.shape
    if not (input_scale > 0.0) or input_scale != input_scale or input_scale == float("inf"):
        raise ShapeError(f"input_scale must be positive and finite, got {input_scale}")
    out = out or Nvfp4Matrix.zeros(tokens, k, x.device)
    if x.dtype == torch.float32:
        _need(x, torch.float32, "activation")
        check("infer_quantize_nvfp4_col_major_f32_on_stream",
              lib.infer_quantize_nvfp4_col_major_f32_on_stream(x.data_ptr(), out.packed.data_ptr(), out.scales.data_ptr(),
                                                               k, tokens, input_scale, _stream()))
    else:
        _need(x, torch.bfloat16, "activation")
        check("eider_b200_quantize_nvfp4_bf16_on_stream",
              lib.eider_b200_quantize_nvfp4_bf16_on_stream(x.data_ptr(), out.packed.data_ptr(), out.scales.data_ptr(), k,
                                                           tokens, input_scale, _stream()))
    return out


def quantize_nvfp4_rowscale(x: torch.Tensor, out: Nvfp4Matrix | None = None) -> Nvfp4Matrix:
    """Per-token global scale g = the smallest power of two >= amax/2688 (1 for an all-zero row), then the reference
    quantizer with input_scale = g; g lands in `row_scales`."""
    lib = _lib.load()
    tokens, k = x.shape
    if x.dtype not in (torch.float32, torch.bfloat16):
        raise ShapeError("activation must be f32 or bf16")
    _need(x, x.dtype, "activation")
    out = out or Nvfp4Matrix.zeros(tokens, k, x.device, row_scales=True)
    check("eider_b200_quantize_nvfp4_rowscale_on_stream",
          lib.eider_b200_quantize_nvfp4_rowscale_on_stream(x.data_ptr(), int(x.dtype == torch.bfloat16),
                                                           out.packed.data_ptr(), out.scales.data_ptr(),
                                                           out.row_scales.data_ptr(), k, tokens, _stream()))
    return out


# ---- weights ------------------------------------------------------------------------------------
@dataclass
class ModelOptWeight:
    """Device NVFP4 weight (crates/eider-cuda/src/modelopt_device.rs:18-22,109-200): the checkpoint's packed
    bytes as they are, row-major scales for the CUDA-core GEMV and tile-repacked scales for the tensor-core
    kernels; matmul_alpha = weight_scale_2 * input_scale."""
    packed: torch.Tensor            # [N, K/2] u8
    scales_row_major: torch.Tensor  # [N, K/16] u8 (checkpoint layout)
    scales_tiled: torch.Tensor      # tiled layout, outer = N
    weight_scale_2: float
    input_scale: float
    out_features: int
    in_features: int

    @property
    def matmul_alpha(self) -> float:
        return self.weight_scale_2 * self.input_scale

    @staticmethod
    def from_checkpoint(packed: torch.Tensor, scales_row_major: torch.Tensor, weight_scale_2: float,
                        input_scale: float = 1.0) -> "ModelOptWeight":
        """Upload-time preparation from ModelOptNvfp4Linear bytes (crates/eider-format/src/modelopt.rs:11-26)."""
        lib = _lib.load()
        n, kh = packed.shape
        k = kh * 2
        if scales_row_major.shape != (n, k // 16):
            raise ShapeError(f"weight_scale must be [{n}, {k // 16}], got {tuple(scales_row_major.shape)}")
        _need(packed, torch.uint8, "weight")
        _need(scales_row_major, torch.uint8, "weight_scale")
        tiled = torch.empty(scale_layout_len(n, k), dtype=torch.uint8, device=packed.device)
        check("eider_b200_nvfp4_scales_to_tiled_on_stream",
              lib.eider_b200_nvfp4_scales_to_tiled_on_stream(scales_row_major.data_ptr(), tiled.data_ptr(), n, k, _stream()))
        return ModelOptWeight(packed, scales_row_major, tiled, float(weight_scale_2), float(input_scale), n, k)

    @staticmethod
    def quantize(weight: torch.Tensor, global_scale: float | None = None, input_scale: float = 1.0) -> "ModelOptWeight":
        """Quantize a dense [N, K] f32/bf16 weight the ModelOpt way: g = amax/(6*448) unless given."""
        lib = _lib.load()
        n, k = weight.shape
        if k % 16 != 0:
            raise ShapeError(f"NVFP4 needs K % 16 == 0, got {k}")
        if weight.dtype not in (torch.float32, torch.bfloat16):
            raise ShapeError("weight must be f32 or bf16")
        _need(weight, weight.dtype, "weight")
        if global_scale is None:
            amax = weight.abs().max().float()
            # one IEEE f32 divide by 6 * 448, 1 for an all-zero weight
            global_scale = float((amax / 2688.0).item()) if float(amax.item()) > 0 else 1.0
        packed = torch.empty(n, k // 2, dtype=torch.uint8, device=weight.device)
        scales = torch.empty(n, k // 16, dtype=torch.uint8, device=weight.device)
        check("eider_b200_quantize_nvfp4_weight_on_stream",
              lib.eider_b200_quantize_nvfp4_weight_on_stream(weight.data_ptr(), int(weight.dtype == torch.bfloat16),
                                                             packed.data_ptr(), scales.data_ptr(), n, k, global_scale,
                                                             _stream()))
        return ModelOptWeight.from_checkpoint(packed, scales, global_scale, input_scale)


# ---- dense GEMM plans -------------------------------------------------------------------------------
class Fp4TnMatmulPlan:
    """Dense W4A4 GEMM plan (crates/eider-cuda/src/cublaslt/fp4_tn.rs:264-796): D = alpha * X . W^T + beta * C with
    fp32 accumulation, BF16 or F32 output [tokens, out_features]."""

    def __init__(self, tokens: int, out_features: int, in_features: int):
        lib = _lib.load()
        if not lib.eider_b200_nvfp4_gemm_tn_supported(tokens, out_features, in_features):
            raise ShapeError(f"unsupported NVFP4 GEMM shape m={tokens} n={out_features} k={in_features}")
        self._lib = lib
        self.m, self.n, self.k = tokens, out_features, in_features
        self._plan = lib.eider_b200_nvfp4_gemm_tn_create(tokens, out_features, in_features)
        if not self._plan:
            raise RuntimeError("eider_b200_nvfp4_gemm_tn_create failed")

    @property
    def block_n(self) -> int:
        """Tile code in use: weight rows per tile, 512 = 256 x 256 tiles on CTA pairs."""
        return int(self._lib.eider_b200_gemm_plan_block_n(self._plan))

    def set_output_peers(self, pointers, ld_out: int) -> None:
        """Fused all-gather: `pointers[q]` = address of this rank's first output column inside rank q's full
        [tokens, ld_out] output (peer memory mapped into this process).  An empty list switches it off."""
        arr = (C.c_void_p * max(1, len(pointers)))(*[C.c_void_p(int(a)) for a in pointers])
        check("eider_b200_gemm_plan_set_output_peers",
              self._lib.eider_b200_gemm_plan_set_output_peers(self._plan, arr, len(pointers), ld_out))

    def set_output_multicast(self, address: int) -> None:
        """Fused all-gather through the switch: `address` = this rank's first output column inside an NVLink multicast
        mapping of every rank's full output (0 switches it off).  Needs set_output_peers first."""
        check("eider_b200_gemm_plan_set_output_multicast",
              self._lib.eider_b200_gemm_plan_set_output_multicast(self._plan, C.c_void_p(int(address)) if address else None))

    def set_block_n(self, block_n: int) -> None:
        if not self._lib.eider_b200_gemm_plan_set_block_n(self._plan, block_n):
            raise ShapeError(f"block_n must be 64, 128, 192, 256, 512 (CTA pairs, 256 x 256) or 384 (CTA pairs, 256 x 192), got {block_n}")

    @property
    def k_splits(self) -> int:
        """K splits in use (1 = none); chosen by the plan for shapes with few tiles and a long K."""
        return int(self._lib.eider_b200_gemm_plan_k_splits(self._plan))

    def set_k_splits(self, splits: int) -> None:
        check("eider_b200_gemm_plan_set_k_splits", self._lib.eider_b200_gemm_plan_set_k_splits(self._plan, splits))

    def run(self, x: Nvfp4Matrix, w: ModelOptWeight, out: torch.Tensor | None = None, alpha: float | None = None,
            beta: float = 0.0, c: torch.Tensor | None = None, out_dtype=torch.bfloat16) -> torch.Tensor:
        if x.rows != self.m or x.k != self.k or w.out_features != self.n or w.in_features != self.k:
            raise ShapeError("operand shapes do not match the plan")
        if out is None:
            out = torch.empty(self.m, self.n, dtype=out_dtype, device=x.packed.device)
        if out.dtype not in (torch.bfloat16, torch.float32) or out.shape != (self.m, self.n) or not out.is_contiguous():
            raise ShapeError("output must be contiguous [tokens, out_features] bf16 or f32")
        if beta != 0.0 and c is None:
            c = out
        a = w.matmul_alpha if alpha is None else alpha
        check("eider_b200_nvfp4_gemm_tn_on_stream",
              self._lib.eider_b200_nvfp4_gemm_tn_on_stream(self._plan, x.packed.data_ptr(), x.scales.data_ptr(),
                                                           w.packed.data_ptr(), w.scales_tiled.data_ptr(), _ptr(c),
                                                           out.data_ptr(), a, beta, _ptr(x.row_scales),
                                                           int(out.dtype == torch.bfloat16), _stream()))
        return out

    def status(self) -> int:
        v = C.c_uint32(0)
        check("eider_b200_gemm_plan_status", self._lib.eider_b200_gemm_plan_status(self._plan, C.byref(v)))
        return v.value

    def close(self) -> None:
        if self._plan:
            self._lib.eider_b200_nvfp4_gemm_tn_destroy(self._plan)
            self._plan = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Fp8TnMatmulPlan:
    """Dense FP8 E4M3 GEMM plan (crates/eider-cuda/src/cublaslt/fp8_tn.rs:13-292) with the per-token and
    per-channel scaling fused into the epilogue."""

    def __init__(self, tokens: int, out_features: int, in_features: int):
        lib = _lib.load()
        if not lib.eider_b200_fp8_gemm_tn_supported(tokens, out_features, in_features):
            raise ShapeError(f"unsupported FP8 GEMM shape m={tokens} n={out_features} k={in_features}")
        self._lib = lib
        self.m, self.n, self.k = tokens, out_features, in_features
        self._plan = lib.eider_b200_fp8_gemm_tn_create(tokens, out_features, in_features)
        if not self._plan:
            raise RuntimeError("eider_b200_fp8_gemm_tn_create failed")

    @property
    def block_n(self) -> int:
        """Tile code in use: weight rows per tile, 512 = 256 x 256 tiles on CTA pairs."""
        return int(self._lib.eider_b200_gemm_plan_block_n(self._plan))

    def set_output_peers(self, pointers, ld_out: int) -> None:
        """Fused all-gather: `pointers[q]` = address of this rank's first output column inside rank q's full
        [tokens, ld_out] output (peer memory mapped into this process).  An empty list switches it off."""
        arr = (C.c_void_p * max(1, len(pointers)))(*[C.c_void_p(int(a)) for a in pointers])
        check("eider_b200_gemm_plan_set_output_peers",
              self._lib.eider_b200_gemm_plan_set_output_peers(self._plan, arr, len(pointers), ld_out))

    def set_output_multicast(self, address: int) -> None:
        """Fused all-gather through the switch: `address` = this rank's first output column inside an NVLink multicast
        mapping of every rank's full output (0 switches it off).  Needs set_output_peers first."""
        check("eider_b200_gemm_plan_set_output_multicast",
              self._lib.eider_b200_gemm_plan_set_output_multicast(self._plan, C.c_void_p(int(address)) if address else None))

    def set_block_n(self, block_n: int) -> None:
        if not self._lib.eider_b200_gemm_plan_set_block_n(self._plan, block_n):
            raise ShapeError(f"block_n must be 64, 128, 192, 256, 512 (CTA pairs, 256 x 256) or 384 (CTA pairs, 256 x 192), got {block_n}")

    @property
    def k_splits(self) -> int:
        """K splits in use (1 = none); chosen by the plan for shapes with few tiles and a long K."""
        return int(self._lib.eider_b200_gemm_plan_k_splits(self._plan))

    def set_k_splits(self, splits: int) -> None:
        check("eider_b200_gemm_plan_set_k_splits", self._lib.eider_b200_gemm_plan_set_k_splits(self._plan, splits))

    def run(self, xq: torch.Tensor, wq: torch.Tensor, token_scale: torch.Tensor | None,
            channel_scale: torch.Tensor | None, out: torch.Tensor | None = None, alpha: float = 1.0, beta: float = 0.0,
            c: torch.Tensor | None = None, out_dtype=torch.bfloat16) -> torch.Tensor:
        if xq.shape != (self.m, self.k) or wq.shape != (self.n, self.k):
            raise ShapeError("operand shapes do not match the plan")
        _need(xq, torch.uint8, "xq")
        _need(wq, torch.uint8, "wq")
        if out is None:
            out = torch.empty(self.m, self.n, dtype=out_dtype, device=xq.device)
        if beta != 0.0 and c is None:
            c = out
        check("eider_b200_fp8_gemm_tn_on_stream",
              self._lib.eider_b200_fp8_gemm_tn_on_stream(self._plan, xq.data_ptr(), wq.data_ptr(), _ptr(c), out.data_ptr(),
                                                         alpha, beta, _ptr(token_scale), _ptr(channel_scale),
                                                         int(out.dtype == torch.bfloat16), _stream()))
        return out

    def status(self) -> int:
        v = C.c_uint32(0)
        check("eider_b200_gemm_plan_status", self._lib.eider_b200_gemm_plan_status(self._plan, C.byref(v)))
        return v.value

    def close(self) -> None:
        if self._plan:
            self._lib.eider_b200_fp8_gemm_tn_destroy(self._plan)
            self._plan = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


# ---- FP8 quantizers ---------------------------------------------------------------------------------
def quantize_fp8_dynamic(x: torch.Tensor):
    """Per-token dynamic E4M3: returns (codes [rows, cols] u8, scales [rows] f32)."""
    lib = _lib.load()
    rows, cols = x.shape
    q = torch.empty(rows, cols, dtype=torch.uint8, device=x.device)
    s = torch.empty(rows, dtype=torch.float32, device=x.device)
    if x.dtype == torch.float32:
        _need(x, torch.float32, "activation")
        check("infer_quantize_fp8_e4m3_dynamic_f32_batch_on_stream",
              lib.infer_quantize_fp8_e4m3_dynamic_f32_batch_on_stream(x.data_ptr(), q.data_ptr(), s.data_ptr(), rows, cols,
                                                                      _stream()))
    else:
        _need(x, torch.bfloat16, "activation")
        check("eider_b200_quantize_fp8_e4m3_dynamic_bf16_batch_on_stream",
              lib.eider_b200_quantize_fp8_e4m3_dynamic_bf16_batch_on_stream(x.data_ptr(), q.data_ptr(), s.data_ptr(), rows,
                                                                            cols, _stream()))
    return q, s


def quantize_fp8_static(x: torch.Tensor, input_scale: float) -> torch.Tensor:
    lib = _lib.load()
    _need(x, torch.float32, "activation")
    q = torch.empty(x.shape, dtype=torch.uint8, device=x.device)
    check("infer_quantize_fp8_e4m3_f32_on_stream",
          lib.infer_quantize_fp8_e4m3_f32_on_stream(x.data_ptr(), q.data_ptr(), x.numel(), input_scale, _stream()))
    return q


def quantize_fp8_weight(w: torch.Tensor):
    """Per-output-channel E4M3 weight: returns (codes [N, K] u8, channel scales [N] f32)."""
    lib = _lib.load()
    n, k = w.shape
    if w.dtype not in (torch.float32, torch.bfloat16):
        raise ShapeError("weight must be f32 or bf16")
    _need(w, w.dtype, "weight")
    q = torch.empty(n, k, dtype=torch.uint8, device=w.device)
    s = torch.empty(n, dtype=torch.float32, device=w.device)
    check("eider_b200_quantize_fp8_weight_on_stream",
          lib.eider_b200_quantize_fp8_weight_on_stream(w.data_ptr(), int(w.dtype == torch.bfloat16), q.data_ptr(),
                                                       s.data_ptr(), n, k, _stream()))
    return q, s


# ---- CUDA-core decode kernels -----------------------------------------------------------------------
def nvfp4_w4a16_matvec(x: torch.Tensor, w: ModelOptWeight, out: torch.Tensor | None = None) -> torch.Tensor:
    """y[b] = weight_scale_2 * W . x[b] with exact f32 products (infer_nvfp4_w4a16_matvec_f32_*).
    x [batch, K] f32 -> f32 out, or bf16 -> bf16 out."""
    lib = _lib.load()
    if x.dim() == 1:
        x = x.unsqueeze(0)
    b, k = x.shape
    if k != w.in_features:
        raise ShapeError(f"in_features mismatch: {k} vs {w.in_features}")
    if out is None:
        out = torch.empty(b, w.out_features, dtype=x.dtype, device=x.device)
    if x.dtype == torch.float32:
        _need(x, torch.float32, "input")
        check("infer_nvfp4_w4a16_matvec_f32_warp_rows_batch_on_stream",
              lib.infer_nvfp4_w4a16_matvec_f32_warp_rows_batch_on_stream(
                  x.data_ptr(), w.packed.data_ptr(), w.scales_row_major.data_ptr(), out.data_ptr(), b, w.out_features,
                  k, w.weight_scale_2, 8, _stream()))
    else:
        _need(x, torch.bfloat16, "input")
        check("eider_b200_nvfp4_w4a16_matvec_bf16_on_stream",
              lib.eider_b200_nvfp4_w4a16_matvec_bf16_on_stream(
                  x.data_ptr(), w.packed.data_ptr(), w.scales_row_major.data_ptr(), out.data_ptr(), b, w.out_features,
                  k, w.weight_scale_2, _stream()))
    return out


def fp8_linear_prequantized_simt(xq: torch.Tensor, s_x: torch.Tensor, wq: torch.Tensor,
                                 channel_scale: torch.Tensor | None, weight_scale: float = 1.0,
                                 out_dtype=torch.float32) -> torch.Tensor:
    lib = _lib.load()
    m, k = xq.shape
    n = wq.shape[0]
    out = torch.empty(m, n, dtype=out_dtype, device=xq.device)
    check("eider_b200_fp8_linear_prequantized_simt_on_stream",
          lib.eider_b200_fp8_linear_prequantized_simt_on_stream(xq.data_ptr(), s_x.data_ptr(), wq.data_ptr(),
                                                                _ptr(channel_scale), weight_scale, out.data_ptr(),
                                                                int(out_dtype == torch.bfloat16), m, n, k, _stream()))
    return out


# ---- tensor-core decode (1..64 tokens) ----------------------------------------------------------------
class Nvfp4DecodeOperand:
    """An activation in the operand form of the decode GEMV (residual NVFP4 terms), written once by the producer of x and read
    by every decode linear that consumes x.  Up to eight bf16 tokens or four f32 tokens."""

    def __init__(self, max_tokens: int, in_features: int):
        lib = _lib.load()
        self._lib = lib
        self.max_tokens, self.k, self.tokens = max_tokens, in_features, 0
        self._op = lib.eider_b200_nvfp4_decode_operand_create(max_tokens, in_features)
        if not self._op:
            raise ShapeError(f"unsupported decode operand tokens<={max_tokens} k={in_features}")

    def expand(self, x: torch.Tensor) -> "Nvfp4DecodeOperand":
        if x.dim() == 1:
            x = x.unsqueeze(0)
        tokens, k = x.shape
        if k != self.k or tokens > self.max_tokens or x.dtype not in (torch.float32, torch.bfloat16):
            raise ShapeError("activation does not match the operand")
        _need(x, x.dtype, "activation")
        check("eider_b200_nvfp4_decode_operand_expand_on_stream",
              self._lib.eider_b200_nvfp4_decode_operand_expand_on_stream(self._op, x.data_ptr(), int(x.dtype == torch.bfloat16),
                                                                         tokens, _stream()))
        self.tokens = tokens
        return self

    def close(self) -> None:
        if self._op:
            self._lib.eider_b200_nvfp4_decode_operand_destroy(self._op)
            self._op = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Nvfp4DecodePlan:
    """W4A16 decode linear on tcgen05: y[t] = weight_scale_2 * W . x[t] for up to 64 tokens.  Plays the role of the
    reference's decode operators (LinearDecodeOp, crates/infer/src/qwen3/infer.rs:3385-3584; Nvfp4DeviceLinear::run_f32_into,
    crates/infer/src/qwen3/qwen36.rs:6399-6460) with the weight matrix streamed once through the tensor cores."""

    def __init__(self, max_tokens: int, out_features: int, in_features: int):
        lib = _lib.load()
        self._lib = lib
        self.max_tokens, self.n, self.k = max_tokens, out_features, in_features
        self._plan = lib.eider_b200_nvfp4_decode_create(max_tokens, out_features, in_features)
        if not self._plan:
            raise ShapeError(f"unsupported decode shape tokens<={max_tokens} n={out_features} k={in_features}")

    def run(self, x: torch.Tensor, w: ModelOptWeight, out: torch.Tensor | None = None, beta: float = 0.0,
            c: torch.Tensor | None = None, out_dtype=torch.bfloat16) -> torch.Tensor:
        if x.dim() == 1:
            x = x.unsqueeze(0)
        tokens, k = x.shape
        if k != self.k or w.in_features != self.k or w.out_features != self.n or tokens > self.max_tokens:
            raise ShapeError("operand shapes do not match the plan")
        if x.dtype not in (torch.float32, torch.bfloat16):
            raise ShapeError("activation must be f32 or bf16")
        _need(x, x.dtype, "activation")
        if out is None:
            out = torch.empty(tokens, self.n, dtype=out_dtype, device=x.device)
        if beta != 0.0 and c is None:
            c = out
        check("eider_b200_nvfp4_w4a16_gemv_on_stream",
              self._lib.eider_b200_nvfp4_w4a16_gemv_on_stream(self._plan, x.data_ptr(), int(x.dtype == torch.bfloat16), tokens,
                                                              w.packed.data_ptr(), w.scales_tiled.data_ptr(),
                                                              w.weight_scale_2, _ptr(c), out.data_ptr(), beta,
                                                              int(out.dtype == torch.bfloat16), _stream()))
        return out

    def run_prepared(self, operand: "Nvfp4DecodeOperand", w: ModelOptWeight, out: torch.Tensor | None = None, beta: float = 0.0,
                     c: torch.Tensor | None = None, out_dtype=torch.bfloat16) -> torch.Tensor:
        """The same linear on an activation its producer has already expanded (Nvfp4DecodeOperand.expand): the GEMV only
        copies its slice of the operand once the kernel before it has finished."""
        if operand.k != self.k or w.in_features != self.k or w.out_features != self.n or not 0 < operand.tokens <= self.max_tokens:
            raise ShapeError("operand shapes do not match the plan")
        if out is None:
            out = torch.empty(operand.tokens, self.n, dtype=out_dtype, device=w.packed.device)
        if beta != 0.0 and c is None:
            c = out
        check("eider_b200_nvfp4_w4a16_gemv_prepared_on_stream",
              self._lib.eider_b200_nvfp4_w4a16_gemv_prepared_on_stream(self._plan, operand._op, w.packed.data_ptr(),
                                                                       w.scales_tiled.data_ptr(), w.weight_scale_2, _ptr(c),
                                                                       out.data_ptr(), beta, int(out.dtype == torch.bfloat16),
                                                                       _stream()))
        return out

    PATHS = {"auto": 0, "stream": 1, "fused": 2, "split": 3, "fused_many": 4}

    def set_path(self, path: str) -> None:
        """Kernel family for a few tokens: "auto" (single-launch tcgen05 kernel, one work item per CTA), "stream" (CUDA-core
        streaming GEMV), "fused" (single-launch kernel, persistent CTAs), "split" (expansion kernel + split-K tcgen05 GEMM),
        "fused_many" (what "auto" picks when the shape allows it)."""
        if not self._lib.eider_b200_decode_plan_set_path(self._plan, self.PATHS[path]):
            raise ShapeError(f"decode path {path!r} was refused")

    def status(self) -> int:
        v = C.c_uint32(0)
        check("eider_b200_decode_plan_status", self._lib.eider_b200_decode_plan_status(self._plan, C.byref(v)))
        return v.value

    def close(self) -> None:
        if self._plan:
            self._lib.eider_b200_decode_destroy(self._plan)
            self._plan = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Fp8DecodePlan:
    """FP8 W8A8 decode linear with per-token dynamic activation scales (Fp8Linear decode path,
    crates/infer/src/qwen3/qwen36.rs:2079-2160) on tcgen05 for up to 64 tokens."""

    def __init__(self, max_tokens: int, out_features: int, in_features: int):
        lib = _lib.load()
        self._lib = lib
        self.max_tokens, self.n, self.k = max_tokens, out_features, in_features
        self._plan = lib.eider_b200_fp8_decode_create(max_tokens, out_features, in_features)
        if not self._plan:
            raise ShapeError(f"unsupported decode shape tokens<={max_tokens} n={out_features} k={in_features}")

    def run(self, x: torch.Tensor, wq: torch.Tensor, channel_scale: torch.Tensor | None, weight_scale: float = 1.0,
            out: torch.Tensor | None = None, out_dtype=torch.bfloat16) -> torch.Tensor:
        if x.dim() == 1:
            x = x.unsqueeze(0)
        tokens, k = x.shape
        if k != self.k or wq.shape != (self.n, self.k) or tokens > self.max_tokens:
            raise ShapeError("operand shapes do not match the plan")
        if x.dtype not in (torch.float32, torch.bfloat16):
            raise ShapeError("activation must be f32 or bf16")
        _need(x, x.dtype, "activation")
        _need(wq, torch.uint8, "weight")
        if out is None:
            out = torch.empty(tokens, self.n, dtype=out_dtype, device=x.device)
        check("eider_b200_fp8_linear_decode_on_stream",
              self._lib.eider_b200_fp8_linear_decode_on_stream(self._plan, x.data_ptr(), int(x.dtype == torch.bfloat16), tokens,
                                                               wq.data_ptr(), _ptr(channel_scale), weight_scale,
                                                               out.data_ptr(), int(out.dtype == torch.bfloat16), _stream()))
        return out

    def run_quantized(self, x_codes: torch.Tensor, x_scale: torch.Tensor, wq: torch.Tensor, channel_scale: torch.Tensor | None,
                      weight_scale: float = 1.0, out: torch.Tensor | None = None, out_dtype=torch.bfloat16) -> torch.Tensor:
        """The same linear on activations their producer has already quantized (E4M3 codes [tokens, k] and one f32 scale per
        token, e.g. from quantize_fp8_dynamic)."""
        tokens, k = x_codes.shape
        if k != self.k or wq.shape != (self.n, self.k) or tokens > self.max_tokens or x_scale.numel() < tokens:
            raise ShapeError("operand shapes do not match the plan")
        _need(x_codes, torch.uint8, "activation codes")
        _need(x_scale, torch.float32, "activation scales")
        _need(wq, torch.uint8, "weight")
        if out is None:
            out = torch.empty(tokens, self.n, dtype=out_dtype, device=x_codes.device)
        check("eider_b200_fp8_linear_decode_quantized_on_stream",
              self._lib.eider_b200_fp8_linear_decode_quantized_on_stream(self._plan, x_codes.data_ptr(), x_scale.data_ptr(), tokens,
                                                                         wq.data_ptr(), _ptr(channel_scale), weight_scale,
                                                                         out.data_ptr(), int(out.dtype == torch.bfloat16), _stream()))
        return out

    def status(self) -> int:
        v = C.c_uint32(0)
        check("eider_b200_decode_plan_status", self._lib.eider_b200_decode_plan_status(self._plan, C.byref(v)))
        return v.value

    def close(self) -> None:
        if self._plan:
            self._lib.eider_b200_decode_destroy(self._plan)
            self._plan = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def rms_norm_quantize_nvfp4(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6, input_scale: float = 1.0) -> "Nvfp4Matrix":
    """Fused RMSNorm -> NVFP4 of [rows, cols] f32 (the reference's infer_rms_norm_quantize_nvfp4_col_major_f32_on_stream)."""
    _need(x, torch.float32, "input")
    _need(weight, torch.float32, "weight")
    rows, cols = x.shape
    if weight.numel() != cols:
        raise ShapeError("weight length must equal the row length")
    out = Nvfp4Matrix.zeros(rows, cols, x.device)
    check("infer_rms_norm_quantize_nvfp4_col_major_f32_on_stream",
          _lib.load().infer_rms_norm_quantize_nvfp4_col_major_f32_on_stream(
              x.data_ptr(), weight.data_ptr(), out.packed.data_ptr(), out.scales.data_ptr(), rows, cols, eps, input_scale,
              _stream()))
    return out


def rms_norm_add_then_rms_norm_quantize_nvfp4(x: torch.Tensor, input_weight: torch.Tensor, residual: torch.Tensor,
                                              quant_weight: torch.Tensor, input_eps: float = 1e-6, quant_eps: float = 1e-6,
                                              input_scale: float = 1.0):
    """h = rmsnorm(x; input_weight) + residual (returned, f32) and NVFP4 of rmsnorm(h; quant_weight) / input_scale
    (the reference's infer_rms_norm_add_then_rms_norm_quantize_nvfp4_f32_on_stream)."""
    for t, name in ((x, "input"), (input_weight, "input_weight"), (residual, "residual"), (quant_weight, "quant_weight")):
        _need(t, torch.float32, name)
    rows, cols = x.shape
    if residual.shape != x.shape or input_weight.numel() != cols or quant_weight.numel() != cols:
        raise ShapeError("operand shapes do not match")
    h = torch.empty_like(x)
    out = Nvfp4Matrix.zeros(rows, cols, x.device)
    check("infer_rms_norm_add_then_rms_norm_quantize_nvfp4_f32_on_stream",
          _lib.load().infer_rms_norm_add_then_rms_norm_quantize_nvfp4_f32_on_stream(
              x.data_ptr(), input_weight.data_ptr(), residual.data_ptr(), h.data_ptr(), quant_weight.data_ptr(),
              out.packed.data_ptr(), out.scales.data_ptr(), rows, cols, input_eps, quant_eps, input_scale, _stream()))
    return h, out


def silu_mul_halves_quantize_nvfp4(gate_up: torch.Tensor, input_scale: float = 1.0) -> "Nvfp4Matrix":
    """Fused SiLU(gate) * up -> NVFP4 of [tokens, 2K] f32 rows (gate half first): the activation of the down projection
    without the fp32 round trip (the reference's infer_silu_mul_halves_quantize_nvfp4_col_major_f32_on_stream)."""
    if gate_up.dim() == 1:
        gate_up = gate_up.unsqueeze(0)
    _need(gate_up, torch.float32, "gate_up")
    tokens, two_k = gate_up.shape
    k = two_k // 2
    if two_k % 32 != 0:
        raise ShapeError("the intermediate size must be a multiple of 16")
    out = Nvfp4Matrix.zeros(tokens, k, gate_up.device)
    check("eider_b200_silu_mul_halves_quantize_nvfp4_batch_on_stream",
          _lib.load().eider_b200_silu_mul_halves_quantize_nvfp4_batch_on_stream(
              gate_up.data_ptr(), out.packed.data_ptr(), out.scales.data_ptr(), tokens, k, input_scale, _stream()))
    return out


def expand_nvfp4_terms(x: torch.Tensor, terms: int):
    """Residual NVFP4 expansion (packed [tokens*terms, K/2], tiled scales, per-row f32 scales)."""
    lib = _lib.load()
    tokens, k = x.shape
    rows = tokens * terms
    packed = torch.zeros(rows, k // 2, dtype=torch.uint8, device=x.device)
    scales = torch.zeros(scale_layout_len(rows, k), dtype=torch.uint8, device=x.device)
    col = torch.zeros(rows, dtype=torch.float32, device=x.device)
    check("eider_b200_expand_nvfp4_terms_on_stream",
          lib.eider_b200_expand_nvfp4_terms_on_stream(x.data_ptr(), int(x.dtype == torch.bfloat16), packed.data_ptr(),
                                                      scales.data_ptr(), col.data_ptr(), tokens, k, terms, _stream()))
    return packed, scales, col


# ---- routed MoE ----------------------------------------------------------------------------------------
def moe_topk(logits: torch.Tensor, k: int, norm_topk_prob: bool):
    """moe_topk_f32_batch (crates/eider-cuda/src/kernels/non_gemm.rs:2131-2196): indices [T, k] u32 (as int32 storage)
    and weights [T, k] f32."""
    lib = _lib.load()
    _need(logits, torch.float32, "logits")
    t, e = logits.shape
    idx = torch.empty(t, k, dtype=torch.int32, device=logits.device)
    w = torch.empty(t, k, dtype=torch.float32, device=logits.device)
    check("infer_moe_topk_f32_batch_on_stream",
          lib.infer_moe_topk_f32_batch_on_stream(logits.data_ptr(), idx.data_ptr(), w.data_ptr(), t, e, k,
                                                 int(bool(norm_topk_prob)), _stream()))
    return idx, w


def moe_scale_tile_bytes(k: int) -> int:
    return 128 * ((k // 16 + 3) // 4 * 4)


class MoeSortedRoutes:
    """Permutation metadata of one MoE layer call (crates/eider-cuda/src/kernels/non_gemm.rs:2199-2323): expert counts,
    offsets [E+1], sorted route ids, sorted expert ids and the inverse map, all device-resident (no host readback)."""

    def __init__(self, routes: int, experts: int, device="cuda"):
        lib = _lib.load()
        self._lib = lib
        self.routes, self.experts = routes, experts
        i32 = dict(dtype=torch.int32, device=device)
        self.expert_counts = torch.zeros(experts, **i32)
        self.expert_offsets = torch.zeros(experts + 1, **i32)
        self.expert_cursors = torch.zeros(experts, **i32)
        self.sorted_routes = torch.zeros(routes, **i32)
        self.sorted_experts = torch.zeros(routes, **i32)
        self.route_to_sorted = torch.zeros(routes, **i32)
        self._scratch = torch.zeros(max(1, lib.eider_b200_moe_sort_scratch_bytes(routes, experts)), dtype=torch.uint8, device=device)

    def sort(self, indices: torch.Tensor) -> "MoeSortedRoutes":
        if indices.numel() != self.routes or indices.dtype != torch.int32:
            raise ShapeError("indices must be int32 with one entry per route")
        check("eider_b200_moe_sort_routes_on_stream",
              self._lib.eider_b200_moe_sort_routes_on_stream(indices.data_ptr(), self.expert_counts.data_ptr(),
                                                             self.expert_offsets.data_ptr(), self.expert_cursors.data_ptr(),
                                                             self.sorted_routes.data_ptr(), self.sorted_experts.data_ptr(),
                                                             self.route_to_sorted.data_ptr(), self.routes, self.experts,
                                                             self._scratch.data_ptr(), self._scratch.numel(), _stream()))
        return self


class MoeSortedNvfp4Rows:
    """Expert-major NVFP4 rows with per-expert 128-row scale tiles (crates/eider-cuda/src/kernels/non_gemm.rs:2326-2821)."""

    def __init__(self, routes: int, experts: int, k: int, tokens: int, device="cuda"):
        self._lib = _lib.load()
        self.routes, self.experts, self.k, self.tokens = routes, experts, k, tokens
        self.tile_bytes = moe_scale_tile_bytes(k)
        self.packed = torch.zeros(routes, k // 2, dtype=torch.uint8, device=device)
        self.scales = torch.zeros(((routes + 127) // 128 + experts) * self.tile_bytes, dtype=torch.uint8, device=device)
        self.source_packed = torch.zeros(tokens, k // 2, dtype=torch.uint8, device=device)
        self.source_scales = torch.zeros(scale_layout_len(tokens, k), dtype=torch.uint8, device=device)

    def gather_quantize(self, x: torch.Tensor, routes: MoeSortedRoutes, routes_per_row: int) -> "MoeSortedNvfp4Rows":
        t, k = x.shape
        if k != self.k or t != self.tokens:
            raise ShapeError("input does not match the buffer")
        name = ("infer_moe_gather_quantize_sorted_routes_nvfp4_on_stream" if x.dtype == torch.float32
                else "eider_b200_moe_gather_quantize_sorted_routes_nvfp4_bf16_on_stream")
        _need(x, x.dtype, "input")
        fn = getattr(self._lib, name)
        check(name, fn(x.data_ptr(), routes.sorted_routes.data_ptr(), routes.sorted_experts.data_ptr(),
                       routes.expert_offsets.data_ptr(), self.source_packed.data_ptr(), self.source_scales.data_ptr(),
                       self.packed.data_ptr(), self.scales.data_ptr(), t, self.routes, routes_per_row, k, self.tile_bytes,
                       _stream()))
        return self

    def silu_mul_halves_quantize(self, gate_up: torch.Tensor, routes: MoeSortedRoutes) -> "MoeSortedNvfp4Rows":
        _need(gate_up, torch.bfloat16, "gate_up")
        if gate_up.shape != (self.routes, 2 * self.k):
            raise ShapeError("gate_up must be [routes, 2 * in_features]")
        check("infer_moe_silu_mul_halves_quantize_sorted_routes_nvfp4_on_stream",
              self._lib.infer_moe_silu_mul_halves_quantize_sorted_routes_nvfp4_on_stream(
                  gate_up.data_ptr(), routes.sorted_experts.data_ptr(), routes.expert_offsets.data_ptr(),
                  self.packed.data_ptr(), self.scales.data_ptr(), self.routes, self.k, self.tile_bytes, _stream()))
        return self


@dataclass
class GroupedNvfp4Weights:
    """Stacked per-expert NVFP4 weights [E, N, K/2] with tiled scales over the stacked [E*N, K] matrix and one
    weight_scale_2 per expert (Qwen36GroupedMoeWeights, crates/infer/src/qwen3/qwen36.rs:3261-3330)."""
    packed: torch.Tensor
    scales_row_major: torch.Tensor
    scales_tiled: torch.Tensor
    alpha: torch.Tensor  # [E] f32
    experts: int
    out_features: int
    in_features: int

    @staticmethod
    def from_checkpoint(packed: torch.Tensor, scales_row_major: torch.Tensor, weight_scale_2: torch.Tensor) -> "GroupedNvfp4Weights":
        e, n, kh = packed.shape
        flat = ModelOptWeight.from_checkpoint(packed.reshape(e * n, kh), scales_row_major.reshape(e * n, kh * 2 // 16), 1.0)
        return GroupedNvfp4Weights(packed, scales_row_major, flat.scales_tiled, weight_scale_2.to(torch.float32).contiguous(),
                                   e, n, kh * 2)

    def interleave_gate_up(self) -> "GroupedNvfp4Weights":
        """The same gate/up weights with the rows of every expert reordered as [16 gate rows, 16 up rows] per 16 features:
        the order the grouped GEMM with the fused SiLU * up quantizer wants (32 consecutive output columns = one
        16-feature block of both halves).  Done once at load."""
        n = self.out_features
        half = n // 2
        if n % 32 != 0:
            raise ShapeError("gate/up rows must come in multiples of 32")
        blocks = torch.arange(half // 16, device=self.packed.device).repeat_interleave(32) * 16
        within = torch.arange(32, device=self.packed.device).repeat(half // 16)
        order = torch.where(within < 16, blocks + within, half + blocks + within - 16)
        return GroupedNvfp4Weights.from_checkpoint(self.packed.index_select(1, order).contiguous(),
                                                   self.scales_row_major.index_select(1, order).contiguous(), self.alpha)

    @staticmethod
    def quantize(weights: torch.Tensor) -> "GroupedNvfp4Weights":
        """[E, N, K] f32/bf16 -> per-expert ModelOpt quantization (own global scale per expert)."""
        e, n, k = weights.shape
        packs, scs, alphas = [], [], []
        for i in range(e):
            w = ModelOptWeight.quantize(weights[i].contiguous())
            packs.append(w.packed)
            scs.append(w.scales_row_major)
            alphas.append(w.weight_scale_2)
        return GroupedNvfp4Weights.from_checkpoint(torch.stack(packs), torch.stack(scs),
                                                   torch.tensor(alphas, dtype=torch.float32, device=weights.device))


class Fp4GroupedGemmPlan:
    """CutlassFp4GroupedGemmPlan (crates/eider-cuda/src/cublaslt/fp4_tn.rs:1160-1278): per expert
    D_e = alpha_e * X_e . W_e^T, bf16 [route, m], token counts stay on the device."""

    def __init__(self, m: int, max_n: int, k: int, groups: int):
        lib = _lib.load()
        if not lib.eider_b200_nvfp4_grouped_gemm_supported(m, max_n, k, groups):
            raise ShapeError(f"unsupported grouped GEMM m={m} k={k} groups={groups}")
        self._lib = lib
        self.m, self.max_n, self.k, self.groups = m, max_n, k, groups
        self._plan = lib.eider_b200_nvfp4_grouped_gemm_create(m, max_n, k, groups)
        if not self._plan:
            raise RuntimeError("eider_b200_nvfp4_grouped_gemm_create failed")

    def run(self, rows: MoeSortedNvfp4Rows, w: GroupedNvfp4Weights, routes: MoeSortedRoutes,
            out: torch.Tensor | None = None) -> torch.Tensor:
        if rows.k != self.k or w.in_features != self.k or w.out_features != self.m or w.experts != self.groups:
            raise ShapeError("operand shapes do not match the plan")
        if out is None:
            out = torch.empty(rows.routes, self.m, dtype=torch.bfloat16, device=rows.packed.device)
        check("eider_b200_nvfp4_grouped_gemm_on_stream",
              self._lib.eider_b200_nvfp4_grouped_gemm_on_stream(self._plan, rows.packed.data_ptr(), rows.scales.data_ptr(),
                                                                w.packed.data_ptr(), w.scales_tiled.data_ptr(), out.data_ptr(),
                                                                w.alpha.data_ptr(), routes.expert_offsets.data_ptr(),
                                                                rows.routes, _stream()))
        return out

    def run_silu_quantize(self, rows: MoeSortedNvfp4Rows, w_interleaved: GroupedNvfp4Weights, routes: MoeSortedRoutes,
                          out: MoeSortedNvfp4Rows) -> MoeSortedNvfp4Rows:
        """Gate/up GEMM with SiLU(gate) * up -> NVFP4 in the epilogue: fills `out` (the down projection's input) without
        materialising the bf16 gate/up rows.  `w_interleaved` = GroupedNvfp4Weights.interleave_gate_up()."""
        if (rows.k != self.k or w_interleaved.in_features != self.k or w_interleaved.out_features != self.m or
                w_interleaved.experts != self.groups or out.k * 2 != self.m or out.routes != rows.routes):
            raise ShapeError("operand shapes do not match the plan")
        check("eider_b200_nvfp4_grouped_gemm_silu_quantize_on_stream",
              self._lib.eider_b200_nvfp4_grouped_gemm_silu_quantize_on_stream(
                  self._plan, rows.packed.data_ptr(), rows.scales.data_ptr(), w_interleaved.packed.data_ptr(),
                  w_interleaved.scales_tiled.data_ptr(), w_interleaved.alpha.data_ptr(), routes.expert_offsets.data_ptr(), rows.routes,
                  out.packed.data_ptr(), out.scales.data_ptr(), out.tile_bytes, _stream()))
        return out

    def status(self) -> int:
        v = C.c_uint32(0)
        check("eider_b200_grouped_plan_status", self._lib.eider_b200_grouped_plan_status(self._plan, C.byref(v)))
        return v.value

    def close(self) -> None:
        if self._plan:
            self._lib.eider_b200_nvfp4_grouped_gemm_destroy(self._plan)
            self._plan = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def moe_weighted_accumulate(routes: MoeSortedRoutes, route_weights: torch.Tensor, sorted_rows: torch.Tensor,
                            tokens: int, routes_per_row: int, out: torch.Tensor | None = None) -> torch.Tensor:
    """moe_weighted_accumulate_sorted_bf16_batch (crates/eider-cuda/src/kernels/non_gemm.rs:3336+): f32 [tokens, len]."""
    lib = _lib.load()
    _need(sorted_rows, torch.bfloat16, "sorted rows")
    _need(route_weights, torch.float32, "route weights")
    ln = sorted_rows.shape[1]
    if out is None:
        out = torch.empty(tokens, ln, dtype=torch.float32, device=sorted_rows.device)
    check("infer_moe_weighted_accumulate_sorted_bf16_batch_on_stream",
          lib.infer_moe_weighted_accumulate_sorted_bf16_batch_on_stream(routes.route_to_sorted.data_ptr(),
                                                                        route_weights.data_ptr(), sorted_rows.data_ptr(),
                                                                        out.data_ptr(), tokens, ln, routes_per_row, _stream()))
    return out


class GroupedMoe:
    """The routed-MoE prefill pipeline of Qwen36MoeWeights::run_batch (crates/infer/src/qwen3/qwen36/batch.rs:6785-6860):
    top-k -> sort -> gather + quantize -> grouped gate/up GEMM -> SiLU * up + quantize -> grouped down GEMM -> combine."""

    def __init__(self, tokens: int, experts: int, top_k: int, hidden: int, intermediate: int, device="cuda"):
        self.tokens, self.experts, self.top_k, self.hidden, self.inter = tokens, experts, top_k, hidden, intermediate
        r = tokens * top_k
        self.routes = MoeSortedRoutes(r, experts, device)
        self.gate_up_in = MoeSortedNvfp4Rows(r, experts, hidden, tokens, device)
        self.down_in = MoeSortedNvfp4Rows(r, experts, intermediate, tokens, device)
        self.gate_up_plan = Fp4GroupedGemmPlan(2 * intermediate, tokens, hidden, experts)
        self.down_plan = Fp4GroupedGemmPlan(hidden, tokens, intermediate, experts)
        self.gate_up_out = torch.empty(r, 2 * intermediate, dtype=torch.bfloat16, device=device)
        self.down_out = torch.empty(r, hidden, dtype=torch.bfloat16, device=device)
        self.out = torch.empty(tokens, hidden, dtype=torch.float32, device=device)

    def run(self, x: torch.Tensor, router_logits: torch.Tensor, w_gate_up: GroupedNvfp4Weights, w_down: GroupedNvfp4Weights,
            norm_topk_prob: bool = True, w_gate_up_interleaved: GroupedNvfp4Weights | None = None) -> torch.Tensor:
        """With `w_gate_up_interleaved` (GroupedNvfp4Weights.interleave_gate_up(), made once at load) the SiLU * up
        quantizer runs in the gate/up GEMM's epilogue and the bf16 gate/up rows never reach HBM; the bytes of the down
        projection's input are the same either way."""
        idx, weights = moe_topk(router_logits, self.top_k, norm_topk_prob)
        self.routes.sort(idx.reshape(-1))
        self.gate_up_in.gather_quantize(x, self.routes, self.top_k)
        if w_gate_up_interleaved is not None:
            self.gate_up_plan.run_silu_quantize(self.gate_up_in, w_gate_up_interleaved, self.routes, self.down_in)
        else:
            self.gate_up_plan.run(self.gate_up_in, w_gate_up, self.routes, out=self.gate_up_out)
            self.down_in.silu_mul_halves_quantize(self.gate_up_out, self.routes)
        self.down_plan.run(self.down_in, w_down, self.routes, out=self.down_out)
        self.route_weights = weights
        self.route_indices = idx
        return moe_weighted_accumulate(self.routes, weights.reshape(-1), self.down_out, self.tokens, self.top_k, out=self.out)


# ---- operator composition ---------------------------------------------------------------------------------
class DenseFfn:
    """The dense gated FFN as the reference composes it for a batch of rows (crates/infer/src/qwen3/qwen36.rs:7175-7280):
    gate_up = X . W_gu^T (W4A4, f32 out) -> SiLU(gate) * up -> NVFP4 with the down projection's static input scale (one
    fused producer) -> down = A . W_d^T with beta = 1 on the residual -> bf16.  GEMM plans are cached by row count, as
    run_nvfp4_batch does (crates/infer/src/qwen3/qwen36/batch.rs:1008-1058), so a new chunk length costs one plan creation
    and a repeated one costs none."""

    def __init__(self, w_gate_up: ModelOptWeight, w_down: ModelOptWeight):
        if w_gate_up.out_features % 2 != 0 or w_down.in_features * 2 != w_gate_up.out_features or w_down.out_features != w_gate_up.in_features:
            raise ShapeError("gate/up must be [2 * intermediate, hidden] and down [hidden, intermediate]")
        self.w_gate_up, self.w_down = w_gate_up, w_down
        self.hidden, self.inter = w_gate_up.in_features, w_down.in_features
        self._plans = {}

    def plans(self, rows: int):
        if rows not in self._plans:
            self._plans[rows] = (Fp4TnMatmulPlan(rows, 2 * self.inter, self.hidden), Fp4TnMatmulPlan(rows, self.hidden, self.inter))
        return self._plans[rows]

    def run(self, x: torch.Tensor, residual: torch.Tensor) -> torch.Tensor:
        """x [rows, hidden] bf16 or f32 (quantized on the fly with a per-row scale), residual [rows, hidden] bf16 -> bf16."""
        rows = x.shape[0]
        if x.shape[1] != self.hidden or residual.shape != (rows, self.hidden) or residual.dtype != torch.bfloat16:
            raise ShapeError("x must be [rows, hidden] and residual bf16 of the same shape")
        gate_up_plan, down_plan = self.plans(rows)
        xq = quantize_nvfp4_rowscale(x)
        gate_up = gate_up_plan.run(xq, self.w_gate_up, out_dtype=torch.float32)
        act = silu_mul_halves_quantize_nvfp4(gate_up, self.w_down.input_scale)
        out = residual.clone()
        return down_plan.run(act, self.w_down, out=out, beta=1.0)  # alpha = weight_scale_2 * input_scale


class DecodeMoe:
    """One decode step of a routed-MoE layer for a single token, through the reference's table-driven entry points
    (crates/eider-cuda/native/non_gemm.cu:13316-13397, 3558-3593, 3823-3845): the experts' weights stay where the
    checkpoint loader put them and are found through device pointer tables; every slot's expert matrix is streamed once."""

    def __init__(self, gate_up: list, down: list, top_k: int):
        """gate_up / down: per-expert ModelOptWeight lists ([2 * intermediate, hidden] and [hidden, intermediate])."""
        lib = _lib.load()
        self._lib = lib
        self.experts, self.top_k = len(gate_up), top_k
        self.hidden, self.inter = gate_up[0].in_features, down[0].in_features
        dev = gate_up[0].packed.device
        table = lambda ts: torch.tensor([t.data_ptr() for t in ts], dtype=torch.int64, device=dev)
        self._keep = (gate_up, down)
        self.gu_w, self.gu_s = table([w.packed for w in gate_up]), table([w.scales_row_major for w in gate_up])
        self.dn_w, self.dn_s = table([w.packed for w in down]), table([w.scales_row_major for w in down])
        self.gu_g = torch.tensor([w.weight_scale_2 for w in gate_up], dtype=torch.float32, device=dev)
        self.dn_g = torch.tensor([w.weight_scale_2 for w in down], dtype=torch.float32, device=dev)
        self.ones = torch.ones(self.experts, dtype=torch.float32, device=dev)
        self.indices = torch.zeros(top_k, dtype=torch.int32, device=dev)
        self.weights = torch.zeros(top_k, dtype=torch.float32, device=dev)
        self.gate_up = torch.zeros(top_k, 2 * self.inter, dtype=torch.float32, device=dev)
        self.act = torch.zeros(top_k, self.inter, dtype=torch.float32, device=dev)
        self.down = torch.zeros(top_k, self.hidden, dtype=torch.float32, device=dev)
        self.gate_up_t, self.act_t, self.down_t = table(list(self.gate_up)), table(list(self.act)), table(list(self.down))
        self.out = torch.zeros(self.hidden, dtype=torch.float32, device=dev)

    def run(self, x: torch.Tensor, router_logits: torch.Tensor, shared_gate_logit: torch.Tensor, shared_output: torch.Tensor,
            residual: torch.Tensor, norm_topk_prob: bool = True) -> torch.Tensor:
        """x [hidden] f32, router_logits [experts] f32; returns residual + routed + sigmoid(shared_gate_logit) * shared_output,
        rounded to bf16 precision (f32 storage), as infer_qwen36_ffn_finalize_routed_f32_on_stream does."""
        lib, s = self._lib, _stream()
        for t, name in ((x, "x"), (router_logits, "router_logits"), (shared_gate_logit, "shared_gate_logit"),
                        (shared_output, "shared_output"), (residual, "residual")):
            _need(t, torch.float32, name)
        check("infer_moe_topk_f32_on_stream", lib.infer_moe_topk_f32_on_stream(router_logits.data_ptr(), self.indices.data_ptr(),
                                                                                self.weights.data_ptr(), self.experts, self.top_k,
                                                                                int(bool(norm_topk_prob)), s))
        check("infer_nvfp4_w4a16_grouped_matvec_f32_on_stream", lib.infer_nvfp4_w4a16_grouped_matvec_f32_on_stream(
            self.indices.data_ptr(), x.data_ptr(), self.gu_w.data_ptr(), self.gu_s.data_ptr(), self.gu_g.data_ptr(), self.gate_up_t.data_ptr(),
            self.experts, self.top_k, 2 * self.inter, self.hidden, s))
        check("infer_moe_silu_slots_f32_on_stream", lib.infer_moe_silu_slots_f32_on_stream(
            self.indices.data_ptr(), self.gate_up_t.data_ptr(), self.act_t.data_ptr(), self.ones.data_ptr(), self.inter, self.top_k, s))
        check("infer_nvfp4_w4a16_grouped_inputs_matvec_f32_on_stream", lib.infer_nvfp4_w4a16_grouped_inputs_matvec_f32_on_stream(
            self.indices.data_ptr(), self.act_t.data_ptr(), self.dn_w.data_ptr(), self.dn_s.data_ptr(), self.dn_g.data_ptr(), self.down_t.data_ptr(),
            self.experts, self.top_k, self.hidden, self.inter, s))
        check("infer_qwen36_ffn_finalize_routed_f32_on_stream", lib.infer_qwen36_ffn_finalize_routed_f32_on_stream(
            self.indices.data_ptr(), self.weights.data_ptr(), self.down_t.data_ptr(), self.ones.data_ptr(), shared_gate_logit.data_ptr(),
            shared_output.data_ptr(), residual.data_ptr(), self.out.data_ptr(), self.hidden, self.top_k, s))
        return self.out
