"""ctypes binding of libeider_b200.so.  There is no fallback: a missing library is an error."""
from __future__ import annotations

import ctypes as C
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "lib", "libeider_b200.so")

_lib = None

_P = C.c_void_p
_U32 = C.c_uint32
_F = C.c_float
_I = C.c_int
_SZ = C.c_size_t
_U64 = C.c_uint64
_S = C.c_char_p

# name -> (restype, argtypes).  Mirrors include/eider_b200.h one to one.
SIGNATURES = {
    "infer_quantize_nvfp4_col_major_f32": (_I, [_P, _P, _P, _U32, _U32, _F]),
    "infer_quantize_nvfp4_col_major_f32_on_stream": (_I, [_P, _P, _P, _U32, _U32, _F, _P]),
    "eider_b200_quantize_nvfp4_bf16_on_stream": (_I, [_P, _P, _P, _U32, _U32, _F, _P]),
    "eider_b200_quantize_nvfp4_rowscale_on_stream": (_I, [_P, _I, _P, _P, _P, _U32, _U32, _P]),
    "eider_b200_quantize_nvfp4_weight_on_stream": (_I, [_P, _I, _P, _P, _U32, _U32, _F, _P]),
    "eider_b200_nvfp4_scales_to_tiled_on_stream": (_I, [_P, _P, _U32, _U32, _P]),
    "eider_b200_nvfp4_scale_layout_len": (_SZ, [_SZ, _SZ]),
    "infer_rms_norm_quantize_nvfp4_col_major_f32_on_stream": (_I, [_P, _P, _P, _P, _U32, _U32, _F, _F, _P]),
    "infer_rms_norm_quantize_nvfp4_pair_col_major_f32_on_stream": (_I, [_P, _P, _P, _P, _P, _P, _U32, _U32, _F, _F, _P]),
    "infer_rms_norm_add_then_rms_norm_quantize_nvfp4_f32_on_stream": (_I, [_P, _P, _P, _P, _P, _P, _P, _U32, _U32, _F, _F, _F, _P]),
    "infer_silu_mul_halves_quantize_nvfp4_col_major_f32_on_stream": (_I, [_P, _P, _P, _U32, _F, _P]),
    "eider_b200_silu_mul_halves_quantize_nvfp4_batch_on_stream": (_I, [_P, _P, _P, _U32, _U32, _F, _P]),
    "infer_rms_norm_f32_on_stream": (_I, [_P, _P, _P, _U32, _U32, _F, _P]),
    "infer_rms_norm_add_f32_on_stream": (_I, [_P, _P, _P, _P, _U32, _U32, _F, _P]),
    "infer_gated_rms_norm_f32_on_stream": (_I, [_P, _P, _P, _P, _U32, _U32, _F, _P]),
    "infer_silu_mul_halves_f32_on_stream": (_I, [_P, _P, _U32, _P]),
    "infer_silu_mul_halves_f32_batch_on_stream": (_I, [_P, _P, _U32, _U32, _P]),
    "infer_gelu_tanh_mul_f32_on_stream": (_I, [_P, _P, _P, _U32, _P]),
    "infer_unpack_heads_f32_on_stream": (_I, [_P, _P, _U32, _U32, _U32, _U32, _P]),
    "infer_gelu_tanh_mul_quantize_nvfp4_col_major_f32_on_stream": (_I, [_P, _P, _P, _P, _U32, _U32, _F, _P]),
    "infer_unpack_heads_quantize_nvfp4_col_major_f32_on_stream": (_I, [_P, _P, _P, _U32, _U32, _U32, _U32, _F, _P]),
    "infer_unpack_heads_quantize_nvfp4_col_major_bf16_on_stream": (_I, [_P, _P, _P, _U32, _U32, _U32, _U32, _F, _P]),
    "infer_gated_rms_norm_quantize_nvfp4_col_major_f32_on_stream": (_I, [_P, _P, _P, _P, _P, _U32, _U32, _U32, _F, _F, _P]),
    "infer_quantize_nvfp4_vector_simple_scales_f32_on_stream": (_I, [_P, _P, _P, _U32, _F, _P]),
    "infer_scale_channel_f32_device_scalar_on_stream": (_I, [_P, _P, _P, _U32, _P]),
    "infer_scale_channel_f32_device_row_scalar_on_stream": (_I, [_P, _P, _P, _U32, _U32, _P]),
    "infer_cutlass_fp4_gemv_f32_supported": (_I, [_U32, _U32]),
    "infer_cutlass_fp4_gemv_f32_on_stream": (_I, [_P, _P, _P, _P, _P, _P, _U32, _U32, _F, _P]),
    "infer_fp8_linear_channel_scaled_dynamic_f32_on_stream": (_I, [_P, _P, _P, _P, _U32, _U32, _P]),
    "infer_fp8_linear_channel_scaled_dynamic_quantized_f32_configured_on_stream": (_I, [_P, _P, _P, _P, _P, _P, _U32, _U32, _U32, _P]),
    "infer_fp8_linear_w8a8_f32_on_stream": (_I, [_P, _P, _P, _U32, _U32, _F, _F, _P]),
    "infer_moe_sort_routes_on_stream": (_I, [_P, _P, _P, _P, _P, _P, _P, _U32, _U32, _P]),
    "infer_moe_quantize_sorted_routes_nvfp4_on_stream": (_I, [_P, _P, _P, _P, _P, _P, _U32, _U32, _U32, _U32, _I, _P]),
    "infer_moe_calibrated_quantize_on_stream": (_I, [_P, _P, _P, _P, _P, _P, _P, _U32, _U32, _U32, _U32, _I, _P]),
    "infer_moe_gelu_tanh_mul_quantize_sorted_routes_nvfp4_on_stream": (_I, [_P, _P, _P, _P, _P, _P, _U32, _U32, _U32, _P]),
    "infer_moe_gather_rms_norm_quantize_sorted_routes_nvfp4_on_stream": (_I, [_P, _P, _P, _P, _P, _P, _P, _P, _P, _U32, _U32, _U32, _U32, _U32, _F, _P]),
    "infer_quantize_fp8_e4m3_dynamic_f32_on_stream": (_I, [_P, _P, _P, _U32, _P]),
    "infer_quantize_fp8_e4m3_dynamic_f32_batch_on_stream": (_I, [_P, _P, _P, _U32, _U32, _P]),
    "eider_b200_quantize_fp8_e4m3_dynamic_bf16_batch_on_stream": (_I, [_P, _P, _P, _U32, _U32, _P]),
    "infer_quantize_fp8_e4m3_f32_on_stream": (_I, [_P, _P, _U32, _F, _P]),
    "eider_b200_quantize_fp8_weight_on_stream": (_I, [_P, _I, _P, _P, _U32, _U32, _P]),
    "infer_nvfp4_w4a16_matvec_f32_on_stream": (_I, [_P, _P, _P, _P, _U32, _U32, _F, _P]),
    "infer_nvfp4_w4a16_matvec_f32_warp_rows_batch_on_stream": (_I, [_P, _P, _P, _P, _U32, _U32, _U32, _F, _U32, _P]),
    "eider_b200_nvfp4_w4a16_matvec_bf16_on_stream": (_I, [_P, _P, _P, _P, _U32, _U32, _U32, _F, _P]),
    "eider_b200_fp8_linear_prequantized_simt_on_stream": (_I, [_P, _P, _P, _P, _F, _P, _I, _U32, _U32, _U32, _P]),
    "eider_b200_nvfp4_gemm_tn_supported": (_I, [_U32, _U32, _U32]),
    "eider_b200_nvfp4_gemm_tn_create": (_P, [_U32, _U32, _U32]),
    "eider_b200_nvfp4_gemm_tn_destroy": (None, [_P]),
    "eider_b200_nvfp4_gemm_tn_on_stream": (_I, [_P, _P, _P, _P, _P, _P, _P, _F, _F, _P, _I, _P]),
    "eider_b200_fp8_gemm_tn_supported": (_I, [_U32, _U32, _U32]),
    "eider_b200_fp8_gemm_tn_create": (_P, [_U32, _U32, _U32]),
    "eider_b200_fp8_gemm_tn_destroy": (None, [_P]),
    "eider_b200_fp8_gemm_tn_on_stream": (_I, [_P, _P, _P, _P, _P, _F, _F, _P, _P, _I, _P]),
    "eider_b200_expand_nvfp4_terms_on_stream": (_I, [_P, _I, _P, _P, _P, _U32, _U32, _U32, _P]),
    "eider_b200_nvfp4_decode_create": (_P, [_U32, _U32, _U32]),
    "eider_b200_fp8_decode_create": (_P, [_U32, _U32, _U32]),
    "eider_b200_decode_destroy": (None, [_P]),
    "eider_b200_decode_plan_status": (_I, [_P, _P]),
    "eider_b200_decode_plan_set_path": (_I, [_P, _U32]),
    "eider_b200_nvfp4_w4a16_gemv_on_stream": (_I, [_P, _P, _I, _U32, _P, _P, _F, _P, _P, _F, _I, _P]),
    "eider_b200_fp8_linear_decode_on_stream": (_I, [_P, _P, _I, _U32, _P, _P, _F, _P, _I, _P]),
    "eider_b200_fp8_linear_decode_quantized_on_stream": (_I, [_P, _P, _P, _U32, _P, _P, _F, _P, _I, _P]),
    "infer_nvfp4_w4a16_matvec_f32_warp_rows_on_stream": (_I, [_P, _P, _P, _P, _U32, _U32, _F, _U32, _P]),
    "infer_nvfp4_w4a16_reuse_matvec_f32_on_stream": (_I, [_P, _P, _P, _P, _P, _P, _P, _P, _U32, _U32, _U32, _U32, _P]),
    "infer_fp8_linear_f32_configured_on_stream": (_I, [_P, _P, _P, _U32, _U32, _F, _U32, _P]),
    "infer_fp8_linear_f32_batch_on_stream": (_I, [_P, _P, _P, _U32, _U32, _U32, _F, _U32, _P]),
    "infer_fp8_linear_pair_f32_configured_on_stream": (_I, [_P, _P, _P, _P, _P, _U32, _U32, _U32, _F, _F, _U32, _P]),
    "infer_fp8_linear_triple_f32_configured_on_stream": (_I, [_P, _P, _P, _P, _P, _P, _P, _U32, _U32, _U32, _U32, _F, _F, _F, _U32, _P]),
    "infer_fp8_linear_channel_scaled_f32_configured_on_stream": (_I, [_P, _P, _P, _P, _U32, _U32, _U32, _P]),
    "infer_fp8_linear_channel_scaled_f32_batch_configured_on_stream": (_I, [_P, _P, _P, _P, _U32, _U32, _U32, _U32, _P]),
    "infer_fp8_linear_channel_scaled_precomputed_dynamic_f32_on_stream": (_I, [_P, _P, _P, _P, _P, _U32, _U32, _P]),
    "infer_silu_mul_halves_clamped_f32_on_stream": (_I, [_P, _P, _U32, _F, _P]),
    "infer_silu_mul_halves_clamped_f32_batch_on_stream": (_I, [_P, _P, _U32, _U32, _F, _P]),
    "infer_fp8_moe_grouped_gate_up_f32_on_stream": (_I, [_P, _P, _P, _P, _P, _P, _P, _P, _U32, _U32, _U32, _P]),
    "infer_moe_silu_quantize_fp8_slots_f32_on_stream": (_I, [_P, _P, _P, _U32, _U32, _P]),
    "infer_fp8_moe_grouped_down_f32_on_stream": (_I, [_P, _P, _P, _P, _P, _P, _U32, _U32, _U32, _P]),
    "infer_cutlass_fp4_grouped_gemm_supported": (_I, [_U32, _U32, _U32, _U32]),
    "infer_cutlass_fp4_grouped_gemm_create": (_P, [_U32, _U32, _U32, _U32]),
    "infer_cutlass_fp4_grouped_gemm_destroy": (None, [_P]),
    "infer_cutlass_fp4_grouped_gemm_on_stream": (_I, [_P, _P, _P, _P, _P, _P, _P, _P, _P]),
    "eider_b200_nvfp4_decode_operand_create": (_P, [_U32, _U32]),
    "eider_b200_nvfp4_decode_operand_destroy": (None, [_P]),
    "eider_b200_nvfp4_decode_operand_expand_on_stream": (_I, [_P, _P, _I, _U32, _P]),
    "eider_b200_nvfp4_w4a16_gemv_prepared_on_stream": (_I, [_P, _P, _P, _P, _F, _P, _P, _F, _I, _P]),
    "infer_moe_topk_f32_on_stream": (_I, [_P, _P, _P, _U32, _U32, _I, _P]),
    "infer_moe_topk_f32_batch_on_stream": (_I, [_P, _P, _P, _U32, _U32, _U32, _I, _P]),
    "eider_b200_moe_sort_scratch_bytes": (_SZ, [_U32, _U32]),
    "eider_b200_moe_sort_routes_on_stream": (_I, [_P, _P, _P, _P, _P, _P, _P, _U32, _U32, _P, _SZ, _P]),
    "eider_b200_moe_sort_routes_noalloc_on_stream": (_I, [_P, _P, _P, _P, _P, _P, _P, _U32, _U32, _P]),
    "eider_b200_moe_sort_noalloc_max_entries": (_SZ, []),
    "infer_moe_gather_quantize_sorted_routes_nvfp4_on_stream": (_I, [_P, _P, _P, _P, _P, _P, _P, _P, _U32, _U32, _U32, _U32, _U32, _P]),
    "eider_b200_moe_gather_quantize_sorted_routes_nvfp4_bf16_on_stream": (_I, [_P, _P, _P, _P, _P, _P, _P, _P, _U32, _U32, _U32, _U32, _U32, _P]),
    "infer_moe_silu_mul_halves_quantize_sorted_routes_nvfp4_on_stream": (_I, [_P, _P, _P, _P, _P, _U32, _U32, _U32, _P]),
    "infer_moe_grouped_pointer_tables_on_stream": (_I, [_P, _P, _P, _P, _P, _P, _P, _U32, _U32, _U32, _U32, _P]),
    "eider_b200_nvfp4_grouped_gemm_supported": (_I, [_U32, _U32, _U32, _U32]),
    "eider_b200_nvfp4_grouped_gemm_create": (_P, [_U32, _U32, _U32, _U32]),
    "eider_b200_nvfp4_grouped_gemm_destroy": (None, [_P]),
    "eider_b200_nvfp4_grouped_gemm_on_stream": (_I, [_P, _P, _P, _P, _P, _P, _P, _P, _U32, _P]),
    "eider_b200_grouped_plan_status": (_I, [_P, _P]),
    "eider_b200_nvfp4_grouped_gemm_silu_quantize_on_stream": (_I, [_P, _P, _P, _P, _P, _P, _P, _U32, _P, _P, _U32, _P]),
    "infer_moe_weighted_accumulate_sorted_bf16_batch_on_stream": (_I, [_P, _P, _P, _P, _U32, _U32, _U32, _P]),
    "eider_b200_gemm_plan_set_block_n": (_I, [_P, _U32]),
    "eider_b200_gemm_plan_block_n": (_U32, [_P]),
    "eider_b200_gemm_plan_set_k_splits": (_I, [_P, _U32]),
    "eider_b200_gemm_plan_k_splits": (_U32, [_P]),
    "eider_b200_gemm_pick_tile": (_U32, [_U32, _U32, _U32]),
    "eider_b200_gemm_pick_k_splits": (_U32, [_I, _U32, _U32, _U32, _U32, _U32]),
    "eider_b200_gemm_plan_set_output_peers": (_I, [_P, _P, _U32, _U32]),
    "eider_b200_gemm_plan_status": (_I, [_P, _P]),
    "eider_b200_gemm_plan_set_output_multicast": (_I, [_P, _P]),
    "eider_b200_peer_barrier_pad_bytes": (_SZ, []),
    "eider_b200_peer_barrier_state_bytes": (_SZ, []),
    "eider_b200_moe_silu_mul_halves_quantize_sorted_routes_nvfp4_limited_on_stream": (_I, [_P, _P, _P, _P, _P, _U32, _U32, _U32, _P, _P]),
    "eider_b200_ep_publish_counts_on_stream": (_I, [_P, _P, _U32, _U32, _U32, _P]),
    "eider_b200_ep_offsets_on_stream": (_I, [_P, _U32, _U32, _U32, _P, _P, _P, _P, _P]),
    "eider_b200_ep_dispatch_rows_on_stream": (_I, [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _U32, _U32, _U32, _U32, _U32, _U32, _U32, _P]),
    "eider_b200_ep_expand_experts_on_stream": (_I, [_P, _U32, _P, _U32, _P]),
    "eider_b200_ep_return_rows_on_stream": (_I, [_P, _P, _P, _P, _U32, _U32, _U32, _P]),
    "eider_b200_nvfp4_artifact_write": (_I, [_S, _S, _U64, _U64, _P, _U64, _P, _U64, _F, _F]),
    "eider_b200_nvfp4_artifact_read_header": (_I, [_S, _P, _P, _P, _P, _P, _P, _P]),
    "eider_b200_nvfp4_artifact_read": (_I, [_S, _P, _U64, _P, _U64, _P, _U64]),
    "eider_b200_compressed_tensors_globals": (_I, [_F, _F, _P, _P]),
    "eider_b200_mxfp4_scales_to_nvfp4": (_I, [_P, _U64, _P]),
    "eider_b200_gguf_nvfp4_unpack": (_I, [_P, _U64, _U64, _U64, _F, _P, _P]),
    "eider_b200_nvfp4_requantize_host": (_I, [_I, _P, _P, _F, _P, _U64, _U64, _P, _P]),
    "eider_b200_nvfp4_scales_to_tiled_host": (None, [_P, _P, _U64, _U64]),
    "eider_b200_prepared_cache_write": (_I, [_S, _U64, _U64, _P, _P, _F]),
    "eider_b200_prepared_cache_matches": (_I, [_S, _U64, _U64]),
    "eider_b200_prepared_cache_read": (_I, [_S, _U64, _U64, _P, _P, _P]),
    "infer_nvfp4_w4a16_grouped_matvec_f32_on_stream": (_I, [_P, _P, _P, _P, _P, _P, _U32, _U32, _U32, _U32, _P]),
    "infer_nvfp4_w4a16_grouped_inputs_matvec_f32_on_stream": (_I, [_P, _P, _P, _P, _P, _P, _U32, _U32, _U32, _U32, _P]),
    "infer_cutlass_fp4_grouped_gemv_f32_supported": (_I, [_U32, _U32, _U32]),
    "infer_cutlass_fp4_grouped_gemv_f32_create": (_P, [_U32, _U32, _U32]),
    "infer_cutlass_fp4_grouped_gemv_f32_destroy": (None, [_P]),
    "infer_cutlass_fp4_grouped_gemv_f32_indexed_a_on_stream": (_I, [_P, _P, _P, _P, _U32, _P, _P, _P, _F, _P]),
    "infer_cutlass_fp4_grouped_gemv_f32_indexed_a_tiled_scales_on_stream": (_I, [_P, _P, _P, _P, _P, _U32, _P, _P, _P, _P, _P]),
    "infer_cutlass_fp4_grouped_gemv_f32_contiguous_b_on_stream": (_I, [_P, _P, _P, _P, _P, _P, _F, _P]),
    "infer_moe_silu_slots_f32_on_stream": (_I, [_P, _P, _P, _P, _U32, _U32, _P]),
    "infer_moe_silu_quantize_slots_nvfp4_simple_scales_on_stream": (_I, [_P, _P, _P, _P, _P, _P, _U32, _U32, _P]),
    "infer_moe_weighted_accumulate_slots_f32_on_stream": (_I, [_P, _P, _P, _P, _P, _U32, _U32, _P]),
    "infer_moe_weighted_accumulate_slots_f32_batch_on_stream": (_I, [_P, _P, _P, _P, _P, _U32, _U32, _U32, _P]),
    "infer_qwen36_ffn_finalize_routed_f32_on_stream": (_I, [_P, _P, _P, _P, _P, _P, _P, _P, _U32, _U32, _P]),
    "infer_qwen36_ffn_finalize_routed_batch_f32_on_stream": (_I, [_P, _P, _P, _P, _P, _P, _P, _P, _U32, _U32, _U32, _P]),
    "infer_nvfp4_w4a16_top1_f32_on_stream": (_I, [_P, _P, _P, _P, _P, _U32, _P, _P, _U32, _U32, _F, _U32, _P]),
    "infer_deepseek4_block_fp8_linear_f32_on_stream": (_I, [_P, _P, _P, _P, _U32, _U32, _U32, _P]),
    "infer_block_fp8_f32_scale_linear_f32_on_stream": (_I, [_P, _P, _P, _P, _U32, _U32, _U32, _P]),
    "eider_b200_peer_barrier_on_stream": (_I, [_P, _U32, _U32, _U32, _P, C.c_uint64, _P]),
}


def load() -> C.CDLL:
    """Load the shared library (building is a separate, explicit step: eider_b200.build)."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m eider_b200.build` "
            "(there is no CPU or PyTorch fallback for this path)")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the symbol is not exported
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


class CudaError(RuntimeError):
    """A C-ABI entry point returned a non-zero cudaError_t (crates/eider-cuda/src/error.rs:8-12)."""

    def __init__(self, name: str, code: int):
        super().__init__(f"{name} failed with cudaError {code}")
        self.name = name
        self.code = code


def check(name: str, code: int) -> None:
    if code != 0:
        raise CudaError(name, int(code))
