/*
 * eider_b200 — C ABI of the B200 (sm_100a) quantized-linear path.
 *
 * This is the boundary the reference binds in crates/eider-cuda/src/ffi.rs: plain C scalars, raw
 * device pointers, a trailing cudaStream_t, cudaError_t results (0 = success).  Conventions kept from
 * the reference (crates/eider-cuda/native/README.md:45-50):
 *   - the caller owns every buffer; pointers are borrowed for the duration of the enqueued work;
 *   - nothing synchronises the device or uses the default stream implicitly;
 *   - null pointers, zero extents and unsupported divisibility return cudaErrorInvalidValue before
 *     any launch; `*_supported` return 1/0; `*_create` return NULL on failure.
 * Symbols named infer_* keep the reference's name and argument list; symbols named eider_b200_* are
 * new or supersede a closed-library call (cuBLASLt / CUTLASS) of the reference, cited per entry.
 *
 * Shapes: tokens = rows of X, in_features = K (reduction), out_features = rows of W.
 * NVFP4 images: values are E2M1 codes packed two per byte (even element in the low nibble),
 * row-major [rows][K/2]; scales are UE4M3 bytes, one per 16 elements, either row-major
 * [rows][K/16] (checkpoint layout) or "tiled" = the 128-row x 4-block layout of
 * crates/eider-cuda/src/format.rs:194-218.
 */
#ifndef EIDER_B200_H
#define EIDER_B200_H

#include <cuda_runtime_api.h>
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define EIDER_B200_API __attribute__((visibility("default")))

/* ---- NVFP4 activation / weight quantizers --------------------------------------------------- */

/* crates/eider-cuda/src/ffi.rs:2363 and :2372 (kernel crates/eider-cuda/native/non_gemm.cu:106-191).
 * input: f32 [cols tokens][rows = K]; packed: [cols][rows/2]; scales: tiled, outer = token. */
EIDER_B200_API cudaError_t infer_quantize_nvfp4_col_major_f32(const float* input, uint8_t* packed, uint8_t* scales,
                                                              uint32_t rows, uint32_t cols, float input_scale);
EIDER_B200_API cudaError_t infer_quantize_nvfp4_col_major_f32_on_stream(const float* input, uint8_t* packed,
                                                                        uint8_t* scales, uint32_t rows, uint32_t cols,
                                                                        float input_scale, cudaStream_t stream);
/* Same operator for bf16 activations (the reference widens bf16 to f32 first, non_gemm.cu:2577). */
EIDER_B200_API cudaError_t eider_b200_quantize_nvfp4_bf16_on_stream(const uint16_t* input, uint8_t* packed,
                                                                    uint8_t* scales, uint32_t rows, uint32_t cols,
                                                                    float input_scale, cudaStream_t stream);
/* On-the-fly quantizer of the prefill GEMM: per token g = the smallest power of two >= amax / 2688 (1 for an all-zero
 * row; a power of two makes the division by g exact), then the operator above with input_scale = g; g is written to
 * row_scales[cols].  Supersedes the static-scale
 * call of crates/eider-cuda/src/modelopt_device.rs:178-194 for inputs without a calibrated scale. */
EIDER_B200_API cudaError_t eider_b200_quantize_nvfp4_rowscale_on_stream(const void* input, int input_is_bf16,
                                                                        uint8_t* packed, uint8_t* scales,
                                                                        float* row_scales, uint32_t rows, uint32_t cols,
                                                                        cudaStream_t stream);
/* Device twin of ModelOptNvfp4Linear::quantize_values (crates/eider-format/src/modelopt.rs:649-716) with a
 * per-tensor global scale: weight [out][in] f32 or bf16 -> packed [out][in/2] + row-major scales [out][in/16]. */
EIDER_B200_API cudaError_t eider_b200_quantize_nvfp4_weight_on_stream(const void* weight, int input_is_bf16,
                                                                      uint8_t* packed, uint8_t* scales_row_major,
                                                                      uint32_t out_features, uint32_t in_features,
                                                                      float global_scale, cudaStream_t stream);
/* Device twin of modelopt_scales_to_cublaslt (crates/eider-format/src/modelopt.rs:1148-1161). */
EIDER_B200_API cudaError_t eider_b200_nvfp4_scales_to_tiled_on_stream(const uint8_t* scales_row_major,
                                                                      uint8_t* scales_tiled, uint32_t out_features,
                                                                      uint32_t in_features, cudaStream_t stream);
/* Residual NVFP4 expansion of up to 64 activation rows for the tensor-core decode GEMV: x ~= sum_j g_j deq(q_j),
 * rows of the result are token * terms + j.  Generalises the reference's residual-term activation quantizer
 * (crates/eider-cuda/native/sm12x_mma.cu:717-880, two residual terms) to `terms` <= 16. */
EIDER_B200_API cudaError_t eider_b200_expand_nvfp4_terms_on_stream(const void* input, int input_is_bf16, uint8_t* packed,
                                                                   uint8_t* scales, float* col_scale, uint32_t tokens,
                                                                   uint32_t in_features, uint32_t terms,
                                                                   cudaStream_t stream);
/* ue4m3_scale_layout_len, crates/eider-cuda/src/format.rs:194-198. */
EIDER_B200_API size_t eider_b200_nvfp4_scale_layout_len(size_t outer, size_t inner);

/* Fused producer RMSNorm -> NVFP4 (crates/eider-cuda/native/non_gemm.cu:193-288): input [rows][cols] f32, weight [cols];
 * value = x * rsqrt(mean(x^2) + eps) * weight / input_scale, then the activation quantizer; scales tiled with outer = row.
 * This implementation needs cols % 16 == 0 and 16-byte aligned input and weight. */
EIDER_B200_API cudaError_t infer_rms_norm_quantize_nvfp4_col_major_f32_on_stream(const float* input, const float* weight,
                                                                                 uint8_t* packed, uint8_t* scales, uint32_t rows,
                                                                                 uint32_t cols, float eps, float input_scale,
                                                                                 cudaStream_t stream);

/* The same with a second, residual NVFP4 term (crates/eider-cuda/native/non_gemm.cu:290-419): residual_packed /
 * residual_scales quantize value - dequantized first term, block by block. */
EIDER_B200_API cudaError_t infer_rms_norm_quantize_nvfp4_pair_col_major_f32_on_stream(
    const float* input, const float* weight, uint8_t* packed, uint8_t* scales, uint8_t* residual_packed, uint8_t* residual_scales,
    uint32_t rows, uint32_t cols, float eps, float input_scale, cudaStream_t stream);

/* Fused producer: post-norm residual add, then the quantizing pre-norm of the next block
 * (crates/eider-cuda/native/non_gemm.cu:746-870).  output = input * rsqrt(mean(input^2) + input_eps) * input_weight +
 * residual (f32, [rows][cols]); packed / scales = NVFP4 of output * rsqrt(mean(output^2) + quant_eps) * quant_weight /
 * input_scale.  This implementation needs cols % 16 == 0, cols <= 12288 and 16-byte aligned f32 operands. */
EIDER_B200_API cudaError_t infer_rms_norm_add_then_rms_norm_quantize_nvfp4_f32_on_stream(
    const float* input, const float* input_weight, const float* residual, float* output, const float* quant_weight,
    uint8_t* packed, uint8_t* scales, uint32_t rows, uint32_t cols, float input_eps, float quant_eps, float input_scale,
    cudaStream_t stream);

/* Fused producer SiLU(gate) * up -> NVFP4 (crates/eider-cuda/src/ffi.rs:2441;
 * crates/eider-cuda/native/non_gemm.cu:559-629): gate_up holds `rows` gate values followed by `rows` up values of one
 * token; packed [rows/2], scales tiled with outer = 0.  This implementation needs rows % 16 == 0 and a 16-byte aligned
 * input.  The batch form takes [tokens][2 * rows] and tiles the scales with outer = token. */
EIDER_B200_API cudaError_t infer_silu_mul_halves_quantize_nvfp4_col_major_f32_on_stream(const float* gate_up, uint8_t* packed,
                                                                                        uint8_t* scales, uint32_t rows,
                                                                                        float input_scale, cudaStream_t stream);
EIDER_B200_API cudaError_t eider_b200_silu_mul_halves_quantize_nvfp4_batch_on_stream(const float* gate_up, uint8_t* packed,
                                                                                     uint8_t* scales, uint32_t tokens,
                                                                                     uint32_t rows, float input_scale,
                                                                                     cudaStream_t stream);

/* Staged halves of the fused producers above: the reference keeps them as separate operators and its tests require
 * fused == staged byte for byte (crates/eider-cuda/src/kernels/non_gemm.rs:19687-19750, 19873-20240); here both halves take
 * every sum and product from the same device functions.
 * crates/eider-cuda/src/ffi.rs:1393 (kernel non_gemm.cu:631-667): output = input * rsqrt(mean(input^2) + eps) * weight. */
EIDER_B200_API cudaError_t infer_rms_norm_f32_on_stream(const float* input, const float* weight, float* output, uint32_t rows,
                                                        uint32_t cols, float eps, cudaStream_t stream);
/* crates/eider-cuda/src/ffi.rs:1402 (kernel non_gemm.cu:700-727): the same plus `residual`. */
EIDER_B200_API cudaError_t infer_rms_norm_add_f32_on_stream(const float* input, const float* weight, const float* residual,
                                                            float* output, uint32_t rows, uint32_t cols, float eps,
                                                            cudaStream_t stream);
/* crates/eider-cuda/src/ffi.rs:3937 (kernel non_gemm.cu:11514-11549): input * inverse_rms * weight * silu(gate). */
EIDER_B200_API cudaError_t infer_gated_rms_norm_f32_on_stream(const float* input, const float* gate, const float* weight,
                                                              float* output, uint32_t rows, uint32_t cols, float eps,
                                                              cudaStream_t stream);
/* crates/eider-cuda/src/ffi.rs:1506 and :1520 (kernel non_gemm.cu:1357-1370): rows of [gate | up] ->
 * (gate / (1 + exp(-gate))) * up, f32 [rows][cols]. */
EIDER_B200_API cudaError_t infer_silu_mul_halves_f32_on_stream(const float* gate_up, float* output, uint32_t len,
                                                               cudaStream_t stream);
EIDER_B200_API cudaError_t infer_silu_mul_halves_f32_batch_on_stream(const float* gate_up, float* output, uint32_t rows,
                                                                     uint32_t cols, cudaStream_t stream);
/* crates/eider-cuda/src/ffi.rs:1492: tanh-approximated GELU(gate) * up over `len` elements. */
/* crates/eider-cuda/src/ffi.rs:1512 and :1527 (kernel non_gemm.cu:1328-1338): the same with gate clamped from above and up
 * clamped to [-limit, limit] first; limit finite and positive. */
EIDER_B200_API cudaError_t infer_silu_mul_halves_clamped_f32_on_stream(const float* gate_up, float* output, uint32_t len,
                                                                       float limit, cudaStream_t stream);
EIDER_B200_API cudaError_t infer_silu_mul_halves_clamped_f32_batch_on_stream(const float* gate_up, float* output, uint32_t rows,
                                                                             uint32_t cols, float limit, cudaStream_t stream);
EIDER_B200_API cudaError_t infer_gelu_tanh_mul_f32_on_stream(const float* gate, const float* up, float* output, uint32_t len,
                                                             cudaStream_t stream);
/* crates/eider-cuda/src/ffi.rs:2873 (kernel non_gemm.cu:8898-8915): attention output [heads][tokens][head_dim] ->
 * token-major rows [output_row_offset + token][heads * head_dim]. */
EIDER_B200_API cudaError_t infer_unpack_heads_f32_on_stream(const float* input, float* output, uint32_t tokens, uint32_t heads,
                                                            uint32_t head_dim, uint32_t output_row_offset, cudaStream_t stream);

/* Fused producer GELU-tanh(gate) * up -> NVFP4 (crates/eider-cuda/src/ffi.rs:2405, kernel non_gemm.cu:421-508): gate and
 * up are [rows][cols] f32.  This implementation needs cols % 16 == 0 and 16-byte aligned gate and up. */
EIDER_B200_API cudaError_t infer_gelu_tanh_mul_quantize_nvfp4_col_major_f32_on_stream(const float* gate, const float* up,
                                                                                      uint8_t* packed, uint8_t* scales,
                                                                                      uint32_t rows, uint32_t cols,
                                                                                      float input_scale, cudaStream_t stream);
/* Fused producer head unpack -> NVFP4 (crates/eider-cuda/src/ffi.rs:2882 and :2893, kernel non_gemm.cu:8951-9060): rows
 * output_row_offset .. output_row_offset + tokens of an NVFP4 matrix with heads * head_dim columns; other rows are not
 * touched.  This implementation needs head_dim % 16 == 0. */
EIDER_B200_API cudaError_t infer_unpack_heads_quantize_nvfp4_col_major_f32_on_stream(const float* input, uint8_t* packed,
                                                                                     uint8_t* scales, uint32_t tokens,
                                                                                     uint32_t heads, uint32_t head_dim,
                                                                                     uint32_t output_row_offset,
                                                                                     float input_scale, cudaStream_t stream);
EIDER_B200_API cudaError_t infer_unpack_heads_quantize_nvfp4_col_major_bf16_on_stream(const uint16_t* input, uint8_t* packed,
                                                                                      uint8_t* scales, uint32_t tokens,
                                                                                      uint32_t heads, uint32_t head_dim,
                                                                                      uint32_t output_row_offset,
                                                                                      float input_scale, cudaStream_t stream);
/* Fused producer per-head gated RMSNorm -> NVFP4 (crates/eider-cuda/src/ffi.rs:3948, kernel non_gemm.cu:12029-12120):
 * head_dim must be 128, as in the reference. */
EIDER_B200_API cudaError_t infer_gated_rms_norm_quantize_nvfp4_col_major_f32_on_stream(
    const float* input, const float* gate, const float* weight, uint8_t* packed, uint8_t* scales, uint32_t rows, uint32_t heads,
    uint32_t head_dim, float eps, float input_scale, cudaStream_t stream);
/* crates/eider-cuda/src/ffi.rs:2415 (kernel non_gemm.cu:510-557): one vector of `rows` values; scales[b] is the scale
 * byte of values 16b .. 16b + 15 in plain order (no tiling). */
EIDER_B200_API cudaError_t infer_quantize_nvfp4_vector_simple_scales_f32_on_stream(const float* input, uint8_t* packed,
                                                                                   uint8_t* scales, uint32_t rows,
                                                                                   float input_scale, cudaStream_t stream);

/* ---- FP8 E4M3 quantizers -------------------------------------------------------------------- */

/* crates/eider-cuda/src/ffi.rs:3198 and :3206 (kernels non_gemm.cu:9952-9974, 10028-10066). */
EIDER_B200_API cudaError_t infer_quantize_fp8_e4m3_dynamic_f32_on_stream(const float* input, uint8_t* quantized_input,
                                                                         float* input_scale, uint32_t cols,
                                                                         cudaStream_t stream);
EIDER_B200_API cudaError_t infer_quantize_fp8_e4m3_dynamic_f32_batch_on_stream(const float* input,
                                                                               uint8_t* quantized_input,
                                                                               float* input_scale, uint32_t rows,
                                                                               uint32_t cols, cudaStream_t stream);
EIDER_B200_API cudaError_t eider_b200_quantize_fp8_e4m3_dynamic_bf16_batch_on_stream(const uint16_t* input,
                                                                                     uint8_t* quantized_input,
                                                                                     float* input_scale, uint32_t rows,
                                                                                     uint32_t cols, cudaStream_t stream);
/* crates/eider-cuda/src/ffi.rs:3278. */
EIDER_B200_API cudaError_t infer_quantize_fp8_e4m3_f32_on_stream(const float* input, uint8_t* output, uint32_t len,
                                                                 float input_scale, cudaStream_t stream);
/* Per-output-channel weight quantizer, s_w[n] = amax_n / 448 (precedent crates/infer/src/qwen3/qwen36.rs:2047-2057). */
EIDER_B200_API cudaError_t eider_b200_quantize_fp8_weight_on_stream(const void* weight, int input_is_bf16, uint8_t* q,
                                                                    float* channel_scale, uint32_t out_features,
                                                                    uint32_t in_features, cudaStream_t stream);

/* crates/eider-cuda/src/ffi.rs:3223 and :3231: in-place values[i] *= channel_scale[i] * scalar[0], and
 * values[r][c] *= channel_scale[c] * row_scale[r].  The fused FP8 plans below apply both scales in their epilogue; these
 * stay for callers that still scale in a separate pass. */
EIDER_B200_API cudaError_t infer_scale_channel_f32_device_scalar_on_stream(float* values, const float* channel_scale,
                                                                           const float* scalar, uint32_t len,
                                                                           cudaStream_t stream);
EIDER_B200_API cudaError_t infer_scale_channel_f32_device_row_scalar_on_stream(float* values, const float* channel_scale,
                                                                               const float* row_scale, uint32_t rows,
                                                                               uint32_t channels, cudaStream_t stream);

/* ---- decode GEMV on CUDA cores (exact f32 semantics of the reference) ------------------------ */

/* crates/eider-cuda/src/ffi.rs:3285 (kernels non_gemm.cu:13147-13256): row-major checkpoint scales. */
EIDER_B200_API cudaError_t infer_nvfp4_w4a16_matvec_f32_on_stream(const float* input, const uint8_t* packed_weight,
                                                                  const uint8_t* weight_scale, float* output,
                                                                  uint32_t out_features, uint32_t in_features,
                                                                  float weight_scale_2, cudaStream_t stream);
/* crates/eider-cuda/src/ffi.rs:3308. */
EIDER_B200_API cudaError_t infer_nvfp4_w4a16_matvec_f32_warp_rows_on_stream(const float* input, const uint8_t* packed_weight,
                                                                            const uint8_t* weight_scale, float* output,
                                                                            uint32_t out_features, uint32_t in_features,
                                                                            float weight_scale_2, uint32_t warps_per_block,
                                                                            cudaStream_t stream); /* ffi.rs:3296 */
EIDER_B200_API cudaError_t infer_nvfp4_w4a16_matvec_f32_warp_rows_batch_on_stream(
    const float* input, const uint8_t* packed_weight, const uint8_t* weight_scale, float* output, uint32_t batch_size,
    uint32_t out_features, uint32_t in_features, float weight_scale_2, uint32_t warps_per_block, cudaStream_t stream);
/* bf16 in / bf16 out form of the same operator. */
EIDER_B200_API cudaError_t eider_b200_nvfp4_w4a16_matvec_bf16_on_stream(const uint16_t* input,
                                                                        const uint8_t* packed_weight,
                                                                        const uint8_t* weight_scale, uint16_t* output,
                                                                        uint32_t batch_size, uint32_t out_features,
                                                                        uint32_t in_features, float weight_scale_2,
                                                                        cudaStream_t stream);
/* FP8 W8A8 for a few pre-quantized tokens, y = (sum xq*w) * s_x[t] * s_w[n]
 * (crates/eider-cuda/src/ffi.rs:3151, kernel non_gemm.cu:9976-10011).  channel_scale may be NULL
 * (then weight_scale is the per-tensor scale). */
EIDER_B200_API cudaError_t eider_b200_fp8_linear_prequantized_simt_on_stream(
    const uint8_t* xq, const float* input_scales, const uint8_t* weight, const float* channel_scale, float weight_scale,
    void* output, int output_is_bf16, uint32_t tokens, uint32_t out_features, uint32_t in_features, cudaStream_t stream);

/* Block-scaled FP8 linears (crates/eider-cuda/native/deepseek4.cu:1457-1495; weights of
 * crates/eider-format/src/modelopt.rs:390-443): weight [rows][cols] E4M3, one scale per 128 x 128 block as an E8M0 byte
 * (first form) or an f32 (second form), f32 activations [batch_rows][cols], f32 output [batch_rows][rows];
 * rows % 128 == 0 and cols % 128 == 0 as in the reference.  CUDA-core streaming kernels: the weight matrix is read once per
 * four tokens. */
EIDER_B200_API cudaError_t infer_deepseek4_block_fp8_linear_f32_on_stream(const float* input, const uint8_t* weight,
                                                                          const uint8_t* scales, float* output, uint32_t batch_rows,
                                                                          uint32_t rows, uint32_t cols, cudaStream_t stream);
EIDER_B200_API cudaError_t infer_block_fp8_f32_scale_linear_f32_on_stream(const float* input, const uint8_t* weight,
                                                                          const float* scales, float* output, uint32_t batch_rows,
                                                                          uint32_t rows, uint32_t cols, cudaStream_t stream);

/* ---- dense GEMM on tcgen05 -------------------------------------------------------------------- */

/* Supersedes cublasLtMatmul behind Fp4TnMatmulPlan (crates/eider-cuda/src/cublaslt/fp4_tn.rs:264-796,
 * crates/eider-cuda/src/ffi.rs:4196).  D[tokens][out] = alpha * token_scale[t] * (X . W^T) + beta * C.
 * m = tokens, n = out features, k = in features (k % 32 == 0).  x_scales / w_scales are tiled. */
EIDER_B200_API int eider_b200_nvfp4_gemm_tn_supported(uint32_t m, uint32_t n, uint32_t k);
EIDER_B200_API void* eider_b200_nvfp4_gemm_tn_create(uint32_t m, uint32_t n, uint32_t k);
EIDER_B200_API void eider_b200_nvfp4_gemm_tn_destroy(void* plan);
EIDER_B200_API cudaError_t eider_b200_nvfp4_gemm_tn_on_stream(void* plan, const uint8_t* x_values,
                                                              const uint8_t* x_scales, const uint8_t* w_values,
                                                              const uint8_t* w_scales, const void* c, void* d,
                                                              float alpha, float beta, const float* token_scale,
                                                              int out_is_bf16, cudaStream_t stream);
/* Supersedes cublasLtMatmul behind Fp8TnMatmulPlan (crates/eider-cuda/src/cublaslt/fp8_tn.rs:13-292) and the
 * separate scaling pass infer_scale_channel_f32_device_row_scalar (crates/eider-cuda/src/ffi.rs:3231):
 * D = alpha * token_scale[t] * channel_scale[n] * (Xq . Wq^T) + beta * C. */
EIDER_B200_API int eider_b200_fp8_gemm_tn_supported(uint32_t m, uint32_t n, uint32_t k);
EIDER_B200_API void* eider_b200_fp8_gemm_tn_create(uint32_t m, uint32_t n, uint32_t k);
EIDER_B200_API void eider_b200_fp8_gemm_tn_destroy(void* plan);
EIDER_B200_API cudaError_t eider_b200_fp8_gemm_tn_on_stream(void* plan, const uint8_t* x_values, const uint8_t* w_values,
                                                            const void* c, void* d, float alpha, float beta,
                                                            const float* token_scale, const float* channel_scale,
                                                            int out_is_bf16, cudaStream_t stream);
/* ---- decode (1..64 tokens) on tcgen05 ---------------------------------------------------------- */

/* Supersedes the decode GEMV family: infer_nvfp4_w4a16_matvec_f32* (crates/eider-cuda/src/ffi.rs:3285-3308, CUDA-core
 * W4A16), infer_cutlass_fp4_gemv_f32_on_stream (crates/eider-cuda/src/ffi.rs:576-588, W4A4) and the sm_121 mma.sync GEMV
 * (crates/eider-cuda/native/sm12x_mma.cu:521-601).  The weight matrix streams through shared memory once (TMA) and the
 * tokens ride on the MMA N dimension; the activation keeps 16-bit accuracy through a residual NVFP4 expansion.
 * y[t][n] = weight_scale_2 * sum_k x[t][k] * w[n][k] (+ beta * c).  The plan owns its scratch (split-K partials,
 * expanded activations); w_scales are tiled. */
EIDER_B200_API void* eider_b200_nvfp4_decode_create(uint32_t max_tokens, uint32_t out_features, uint32_t in_features);
EIDER_B200_API cudaError_t eider_b200_nvfp4_w4a16_gemv_on_stream(void* plan, const void* input, int input_is_bf16,
                                                                 uint32_t tokens, const uint8_t* w_values,
                                                                 const uint8_t* w_scales_tiled, float weight_scale_2,
                                                                 const void* c, void* d, float beta, int out_is_bf16,
                                                                 cudaStream_t stream);
/* The same GEMV with the residual expansion of x taken out of its dependency chain: the producer of x expands it once into
 * an operand object (packed term rows, scale bytes and row scales in the layout the GEMV copies straight into shared
 * memory), and every GEMV that consumes x (q/k/v, gate/up) only copies its K slice after the kernel before it has
 * finished.  Up to eight bf16 tokens (four terms each) or four f32 tokens (eight terms) per operand.  No reference
 * counterpart: the reference's W4A16 GEMV reads f32 x directly (crates/eider-cuda/src/ffi.rs:3285-3308).  The operand
 * records the token count of its last expansion; expansion and the GEMVs that read it run in stream order. */
EIDER_B200_API void* eider_b200_nvfp4_decode_operand_create(uint32_t max_tokens, uint32_t in_features);
EIDER_B200_API void eider_b200_nvfp4_decode_operand_destroy(void* operand);
EIDER_B200_API cudaError_t eider_b200_nvfp4_decode_operand_expand_on_stream(void* operand, const void* input,
                                                                            int input_is_bf16, uint32_t tokens,
                                                                            cudaStream_t stream);
EIDER_B200_API cudaError_t eider_b200_nvfp4_w4a16_gemv_prepared_on_stream(void* plan, const void* operand,
                                                                          const uint8_t* w_values,
                                                                          const uint8_t* w_scales_tiled,
                                                                          float weight_scale_2, const void* c, void* d,
                                                                          float beta, int out_is_bf16,
                                                                          cudaStream_t stream);
/* Supersedes infer_fp8_linear_channel_scaled_dynamic_f32_on_stream and its batch forms
 * (crates/eider-cuda/src/ffi.rs:3110-3162; kernels non_gemm.cu:9826-10011): per-token dynamic E4M3 activations,
 * per-channel (channel_scale != NULL) or per-tensor (weight_scale) weight scales. */
EIDER_B200_API void* eider_b200_fp8_decode_create(uint32_t max_tokens, uint32_t out_features, uint32_t in_features);
EIDER_B200_API cudaError_t eider_b200_fp8_linear_decode_on_stream(void* plan, const void* input, int input_is_bf16,
                                                                  uint32_t tokens, const uint8_t* weight,
                                                                  const float* channel_scale, float weight_scale, void* d,
                                                                  int out_is_bf16, cudaStream_t stream);
/* The same linear on activations that are already E4M3 codes [tokens][in_features] with one scale per token: the output
 * of the per-token quantizer (infer_quantize_fp8_e4m3_dynamic_f32_batch_on_stream, crates/eider-cuda/src/ffi.rs:3206),
 * run by the producer of x.  The call above is this one behind that quantizer.  No reference counterpart as an entry
 * point: the reference's FP8 linears quantize inside (crates/eider-cuda/native/non_gemm.cu:9826-10011). */
EIDER_B200_API cudaError_t eider_b200_fp8_linear_decode_quantized_on_stream(void* plan, const uint8_t* x_codes,
                                                                            const float* x_scale, uint32_t tokens,
                                                                            const uint8_t* weight, const float* channel_scale,
                                                                            float weight_scale, void* d, int out_is_bf16,
                                                                            cudaStream_t stream);
EIDER_B200_API void eider_b200_decode_destroy(void* plan);
EIDER_B200_API cudaError_t eider_b200_decode_plan_status(void* plan, uint32_t* host_status);
/* Kernel family for a few tokens of an NVFP4 decode plan: 0 = automatic (the single-launch tcgen05 kernel, one work item
 * per CTA, for up to three bf16 or two f32 tokens; the expansion kernel + split-K tcgen05 GEMM beyond), 1 = CUDA-core
 * streaming GEMV (one or two tokens), 2 = single-launch tcgen05 kernel with persistent CTAs, 3 = expansion kernel + split-K
 * tcgen05 GEMM always, 4 = single-launch kernel with one work item per CTA.  Returns 1 on success. */
EIDER_B200_API int eider_b200_decode_plan_set_path(void* plan, uint32_t path);

/* Plan-less entry points of the reference, served by the kernels above through plans the library keeps per (device, out
 * features, in features).  The first call with a shape allocates its plan and must come before any stream capture; calls
 * with the same shape share the plan's scratch and must not overlap on one GPU.  in_features % 16 == 0 (FP8), % 32 (NVFP4).
 * crates/eider-cuda/src/ffi.rs:576-588 (crates/eider-cuda/native/cutlass_gemv.cu:165-243): W4A4 GEMV with F32 output,
 * d[m] = alpha * sum_k a[m][k] * b[k]; a = weight rows, b = one NVFP4 activation row, both with tiled scales; c must be
 * non-null as in the reference and is not read. */
EIDER_B200_API int infer_cutlass_fp4_gemv_f32_supported(uint32_t m, uint32_t k);
EIDER_B200_API cudaError_t infer_cutlass_fp4_gemv_f32_on_stream(const uint8_t* a_values, const uint8_t* a_scales,
                                                                const uint8_t* b_values, const uint8_t* b_scales, const float* c,
                                                                float* d, uint32_t m, uint32_t k, float alpha,
                                                                cudaStream_t stream);
/* crates/eider-cuda/src/ffi.rs:3131, :3151 and :3239 (kernels non_gemm.cu:9826-10011): one token, rows = out features,
 * cols = in features. */
EIDER_B200_API cudaError_t infer_fp8_linear_channel_scaled_dynamic_f32_on_stream(const float* input, const uint8_t* weight,
                                                                                 const float* channel_weight_scale,
                                                                                 float* output, uint32_t rows, uint32_t cols,
                                                                                 cudaStream_t stream);
EIDER_B200_API cudaError_t infer_fp8_linear_channel_scaled_dynamic_quantized_f32_configured_on_stream(
    const float* input, uint8_t* quantized_input, const uint8_t* weight, const float* channel_weight_scale, float* input_scale,
    float* output, uint32_t rows, uint32_t cols, uint32_t threads, cudaStream_t stream);
/* crates/eider-cuda/src/ffi.rs:3163, :3177 and :3185 (kernels non_gemm.cu:10156-10350): the decode-side routed MoE on FP8
 * experts.  gate_up: every slot multiplies the one E4M3 activation row (scale input_scale[0]) by its expert's gate and up
 * matrices [rows][cols] (per-row scales) into output[slot][gate rows | up rows]; silu_quantize: SiLU(gate) * up per slot with
 * one dynamic scale per slot (amax / 448) into E4M3 codes [slots][rows]; down: every slot multiplies its own code row
 * (scale input_scales[slot]) by its expert's matrix into outputs[slot].  cols % 16 == 0 and 16-byte aligned weights here. */
EIDER_B200_API cudaError_t infer_fp8_moe_grouped_gate_up_f32_on_stream(const uint32_t* indices, const uint8_t* input,
                                                                       const float* input_scale, const uint8_t* const* gate_weights,
                                                                       const float* const* gate_scales,
                                                                       const uint8_t* const* up_weights, const float* const* up_scales,
                                                                       float* output, uint32_t rows, uint32_t cols, uint32_t slots,
                                                                       cudaStream_t stream);
EIDER_B200_API cudaError_t infer_moe_silu_quantize_fp8_slots_f32_on_stream(const float* gate_up, uint8_t* quantized, float* scales,
                                                                           uint32_t rows, uint32_t slots, cudaStream_t stream);
EIDER_B200_API cudaError_t infer_fp8_moe_grouped_down_f32_on_stream(const uint32_t* indices, const uint8_t* inputs,
                                                                    const float* input_scales, const uint8_t* const* weights,
                                                                    const float* const* weight_scales, float* const* outputs,
                                                                    uint32_t rows, uint32_t cols, uint32_t slots,
                                                                    cudaStream_t stream);
/* crates/eider-cuda/src/ffi.rs:3056-3147 (kernels non_gemm.cu:9642-9950): FP8 weight-only linears, f32 activations times
 * E4M3 weights [rows][cols], one weight scale or one per output row; `batch` forms take [batch][cols] inputs and write
 * [batch][rows]; the pair / triple forms run two / three weights on one input.  The "precomputed dynamic" form first writes
 * input_scale[0] = amax(input) / 448 (1 for an all-zero input) and then multiplies e4m3(input / input_scale) by the weights.
 * cols % 16 == 0 and 16-byte aligned weights here; `threads` is validated as in the reference (64..512, multiple of 32)
 * and otherwise unused. */
EIDER_B200_API cudaError_t infer_fp8_linear_f32_configured_on_stream(const float* input, const uint8_t* weight, float* output,
                                                                     uint32_t rows, uint32_t cols, float weight_scale,
                                                                     uint32_t threads, cudaStream_t stream);
EIDER_B200_API cudaError_t infer_fp8_linear_f32_batch_on_stream(const float* input, const uint8_t* weight, float* output,
                                                                uint32_t batch_size, uint32_t rows, uint32_t cols,
                                                                float weight_scale, uint32_t threads, cudaStream_t stream);
EIDER_B200_API cudaError_t infer_fp8_linear_pair_f32_configured_on_stream(const float* input, const uint8_t* first_weight,
                                                                          const uint8_t* second_weight, float* first_output,
                                                                          float* second_output, uint32_t first_rows,
                                                                          uint32_t second_rows, uint32_t cols, float first_scale,
                                                                          float second_scale, uint32_t threads,
                                                                          cudaStream_t stream);
EIDER_B200_API cudaError_t infer_fp8_linear_triple_f32_configured_on_stream(
    const float* input, const uint8_t* first_weight, const uint8_t* second_weight, const uint8_t* third_weight, float* first_output,
    float* second_output, float* third_output, uint32_t first_rows, uint32_t second_rows, uint32_t third_rows, uint32_t cols,
    float first_scale, float second_scale, float third_scale, uint32_t threads, cudaStream_t stream);
EIDER_B200_API cudaError_t infer_fp8_linear_channel_scaled_f32_configured_on_stream(const float* input, const uint8_t* weight,
                                                                                    const float* channel_weight_scale,
                                                                                    float* output, uint32_t rows, uint32_t cols,
                                                                                    uint32_t threads, cudaStream_t stream);
EIDER_B200_API cudaError_t infer_fp8_linear_channel_scaled_f32_batch_configured_on_stream(
    const float* input, const uint8_t* weight, const float* channel_weight_scale, float* output, uint32_t batch_size, uint32_t rows,
    uint32_t cols, uint32_t threads, cudaStream_t stream);
EIDER_B200_API cudaError_t infer_fp8_linear_channel_scaled_precomputed_dynamic_f32_on_stream(
    const float* input, const uint8_t* weight, const float* channel_weight_scale, float* input_scale, float* output, uint32_t rows,
    uint32_t cols, cudaStream_t stream);
EIDER_B200_API cudaError_t infer_fp8_linear_w8a8_f32_on_stream(const float* input, const uint8_t* weight, float* output,
                                                               uint32_t rows, uint32_t cols, float weight_scale,
                                                               float input_scale, cudaStream_t stream);

/* ---- routed MoE ----------------------------------------------------------------------------------- */

/* crates/eider-cuda/src/ffi.rs:1638 and :1691 (kernel non_gemm.cu:1854-2020): softmax / top-k router. */
EIDER_B200_API cudaError_t infer_moe_topk_f32_on_stream(const float* logits, uint32_t* out_indices, float* out_weights,
                                                        uint32_t experts, uint32_t k, int norm_topk_prob,
                                                        cudaStream_t stream);
EIDER_B200_API cudaError_t infer_moe_topk_f32_batch_on_stream(const float* logits, uint32_t* out_indices,
                                                              float* out_weights, uint32_t batch_size, uint32_t experts,
                                                              uint32_t k, int norm_topk_prob, cudaStream_t stream);
/* Supersedes infer_moe_sort_routes_on_stream (crates/eider-cuda/src/ffi.rs:1701, kernels non_gemm.cu:2473-2550): same
 * outputs, but routes of one expert keep ascending route order (the reference's atomic scatter leaves that order
 * unspecified), which needs `scratch` of eider_b200_moe_sort_scratch_bytes(routes, experts) bytes. */
EIDER_B200_API size_t eider_b200_moe_sort_scratch_bytes(uint32_t routes, uint32_t experts);
EIDER_B200_API cudaError_t eider_b200_moe_sort_routes_on_stream(const uint32_t* indices, uint32_t* expert_counts,
                                                                uint32_t* expert_offsets, uint32_t* expert_cursors,
                                                                uint32_t* sorted_routes, uint32_t* sorted_experts,
                                                                uint32_t* route_to_sorted, uint32_t routes, uint32_t experts,
                                                                void* scratch, size_t scratch_bytes, cudaStream_t stream);
/* No counterpart in the reference.  The same route sort for callers that can neither pass scratch nor allocate: a
 * binding that only has the seven output buffers of the reference's sort call to offer, or an engine whose memory plan
 * is frozen after model load and whose step loop is forbidden to call the allocator (an allocation there would fail a
 * stream capture or break the budget).  The chunk histograms live in a 1 MiB table inside the library image instead, so
 * ceil(routes / 256) * experts must not exceed eider_b200_moe_sort_noalloc_max_entries() (262144; larger requests return
 * cudaErrorInvalidValue).  The first call on each device resolves the table's address and should come before any stream
 * capture; calls that overlap on one GPU share the table and race. */
EIDER_B200_API cudaError_t eider_b200_moe_sort_routes_noalloc_on_stream(const uint32_t* indices, uint32_t* expert_counts,
                                                                        uint32_t* expert_offsets, uint32_t* expert_cursors,
                                                                        uint32_t* sorted_routes, uint32_t* sorted_experts,
                                                                        uint32_t* route_to_sorted, uint32_t routes,
                                                                        uint32_t experts, cudaStream_t stream);
EIDER_B200_API size_t eider_b200_moe_sort_noalloc_max_entries(void);
/* crates/eider-cuda/src/ffi.rs:1701 (kernels non_gemm.cu:2473-2550): the reference's sort call as it is, without scratch.
 * It runs the stable sort above through the table inside the library, so it has the same limit on ceil(routes / 256) *
 * experts and the same rules (first call per device before any capture, no overlapping sorts on one GPU). */
EIDER_B200_API cudaError_t infer_moe_sort_routes_on_stream(const uint32_t* indices, uint32_t* expert_counts,
                                                           uint32_t* expert_offsets, uint32_t* expert_cursors,
                                                           uint32_t* sorted_routes, uint32_t* sorted_experts,
                                                           uint32_t* route_to_sorted, uint32_t routes, uint32_t experts,
                                                           cudaStream_t stream);
/* crates/eider-cuda/src/ffi.rs:1728 (kernel non_gemm.cu:2621-2700): quantize sorted rows straight from f32 rows (unit
 * global scale); row of sorted route s = gather_rows ? sorted_routes[s] / routes_per_row : s.  in_features % 16 == 0. */
EIDER_B200_API cudaError_t infer_moe_quantize_sorted_routes_nvfp4_on_stream(
    const float* input, const uint32_t* sorted_routes, const uint32_t* sorted_experts, const uint32_t* expert_offsets,
    uint8_t* packed, uint8_t* scales, uint32_t routes, uint32_t routes_per_row, uint32_t in_features, uint32_t scale_tile_bytes,
    int gather_rows, cudaStream_t stream);
/* crates/eider-cuda/src/ffi.rs:1713 (kernel non_gemm.cu:2562-2619): per-expert calibrated scales, value = x * (1 /
 * input_scales[expert]); relu_squared = 0: f32 token rows gathered by route; 1: sorted bf16 rows, max(x, 0)^2 first. */
EIDER_B200_API cudaError_t infer_moe_calibrated_quantize_on_stream(
    const void* input, const float* input_scales, const uint32_t* sorted_routes, const uint32_t* sorted_experts,
    const uint32_t* expert_offsets, uint8_t* packed, uint8_t* scales, uint32_t routes, uint32_t routes_per_row,
    uint32_t features, uint32_t scale_tile_bytes, int relu_squared, cudaStream_t stream);
/* crates/eider-cuda/src/ffi.rs:1742 (kernel non_gemm.cu:2705-2803): GELU-tanh(gate) * up of sorted bf16 rows. */
EIDER_B200_API cudaError_t infer_moe_gelu_tanh_mul_quantize_sorted_routes_nvfp4_on_stream(
    const uint16_t* gate, const uint16_t* up, const uint32_t* sorted_experts, const uint32_t* expert_offsets, uint8_t* packed,
    uint8_t* scales, uint32_t routes, uint32_t in_features, uint32_t scale_tile_bytes, cudaStream_t stream);
/* crates/eider-cuda/src/ffi.rs:1765 (kernel non_gemm.cu:3000-3064): RMSNorm each token once, quantize it (unit scale)
 * into source_packed / source_scales, then scatter as the gather + quantize call below does. */
EIDER_B200_API cudaError_t infer_moe_gather_rms_norm_quantize_sorted_routes_nvfp4_on_stream(
    const float* input, const float* weight, const uint32_t* sorted_routes, const uint32_t* sorted_experts,
    const uint32_t* expert_offsets, uint8_t* source_packed, uint8_t* source_scales, uint8_t* packed, uint8_t* scales,
    uint32_t rows, uint32_t routes, uint32_t routes_per_row, uint32_t in_features, uint32_t scale_tile_bytes, float eps,
    cudaStream_t stream);
/* crates/eider-cuda/src/ffi.rs:1783 (kernels non_gemm.cu:2899-2998): quantize each token once (unit global scale) into
 * source_packed / source_scales, then scatter the bytes into expert-major rows and per-expert 128-row scale tiles. */
EIDER_B200_API cudaError_t infer_moe_gather_quantize_sorted_routes_nvfp4_on_stream(
    const float* input, const uint32_t* sorted_routes, const uint32_t* sorted_experts, const uint32_t* expert_offsets,
    uint8_t* source_packed, uint8_t* source_scales, uint8_t* packed, uint8_t* scales, uint32_t rows, uint32_t routes,
    uint32_t routes_per_row, uint32_t in_features, uint32_t scale_tile_bytes, cudaStream_t stream);
EIDER_B200_API cudaError_t eider_b200_moe_gather_quantize_sorted_routes_nvfp4_bf16_on_stream(
    const uint16_t* input, const uint32_t* sorted_routes, const uint32_t* sorted_experts, const uint32_t* expert_offsets,
    uint8_t* source_packed, uint8_t* source_scales, uint8_t* packed, uint8_t* scales, uint32_t rows, uint32_t routes,
    uint32_t routes_per_row, uint32_t in_features, uint32_t scale_tile_bytes, cudaStream_t stream);
/* crates/eider-cuda/src/ffi.rs:1754 (kernel non_gemm.cu:2805-2897). */
EIDER_B200_API cudaError_t infer_moe_silu_mul_halves_quantize_sorted_routes_nvfp4_on_stream(
    const uint16_t* gate_up, const uint32_t* sorted_experts, const uint32_t* expert_offsets, uint8_t* packed, uint8_t* scales,
    uint32_t routes, uint32_t in_features, uint32_t scale_tile_bytes, cudaStream_t stream);
/* The same with a device-resident row count: rows at or beyond *routes_limit are skipped (`routes` is then the capacity the
 * launch is sized for).  For buffers whose fill level only the device knows, as in the expert-parallel path below. */
EIDER_B200_API cudaError_t eider_b200_moe_silu_mul_halves_quantize_sorted_routes_nvfp4_limited_on_stream(
    const uint16_t* gate_up, const uint32_t* sorted_experts, const uint32_t* expert_offsets, uint8_t* packed, uint8_t* scales,
    uint32_t routes, uint32_t in_features, uint32_t scale_tile_bytes, const uint32_t* routes_limit, cudaStream_t stream);
/* crates/eider-cuda/src/ffi.rs:1799 (kernel non_gemm.cu:3066-3110). */
EIDER_B200_API cudaError_t infer_moe_grouped_pointer_tables_on_stream(const uint32_t* expert_offsets, const uint8_t* packed,
                                                                      const uint8_t* scales, uint16_t* output,
                                                                      const uint8_t** packed_table, const uint8_t** scale_table,
                                                                      uint16_t** output_table, uint32_t experts,
                                                                      uint32_t in_features, uint32_t out_features,
                                                                      uint32_t scale_tile_bytes, cudaStream_t stream);
/* Supersedes infer_cutlass_fp4_grouped_gemm_{supported,create,destroy,on_stream} (crates/eider-cuda/src/ffi.rs:643-667):
 * per expert e, rows [offsets[e], offsets[e+1]) of a_values times W_e^T, scaled by alpha[e], bf16 output [route][m].
 * w_values is [groups][m][k/2], w_scales_tiled the tiled scales of the stacked [groups*m][k] matrix, a_scales the
 * per-expert tile ranges the quantizers above write. */
EIDER_B200_API int eider_b200_nvfp4_grouped_gemm_supported(uint32_t m, uint32_t max_n, uint32_t k, uint32_t groups);
EIDER_B200_API void* eider_b200_nvfp4_grouped_gemm_create(uint32_t m, uint32_t max_n, uint32_t k, uint32_t groups);
EIDER_B200_API void eider_b200_nvfp4_grouped_gemm_destroy(void* plan);
EIDER_B200_API cudaError_t eider_b200_nvfp4_grouped_gemm_on_stream(void* plan, const uint8_t* a_values,
                                                                   const uint8_t* a_scales, const uint8_t* w_values,
                                                                   const uint8_t* w_scales_tiled, uint16_t* output,
                                                                   const float* alpha, const uint32_t* expert_offsets,
                                                                   uint32_t total_routes, cudaStream_t stream);
/* The gate/up grouped GEMM with SiLU(gate) * up -> NVFP4 in its epilogue: what infer_cutlass_fp4_grouped_gemm_on_stream
 * followed by infer_moe_silu_mul_halves_quantize_sorted_routes_nvfp4_on_stream compute, byte for byte, without the bf16
 * [route][2 * intermediate] round trip through HBM.  The plan's m is 2 * intermediate; the weight rows of every expert must
 * be interleaved as [16 gate rows, 16 up rows] per 16 features (and the scales tiled over that order).  packed
 * [route][intermediate / 2] (16-byte aligned, intermediate % 32 == 0) and scales (per-expert 128-row tiles of
 * scale_tile_bytes) are the down projection's input. */
EIDER_B200_API cudaError_t eider_b200_nvfp4_grouped_gemm_silu_quantize_on_stream(
    void* plan, const uint8_t* a_values, const uint8_t* a_scales, const uint8_t* w_values_interleaved,
    const uint8_t* w_scales_tiled_interleaved, const float* alpha, const uint32_t* expert_offsets, uint32_t total_routes,
    uint8_t* packed, uint8_t* scales, uint32_t scale_tile_bytes, cudaStream_t stream);
/* crates/eider-cuda/src/ffi.rs:643-667 (CutlassFp4GroupedGemmPlan, crates/eider-cuda/src/cublaslt/fp4_tn.rs:1160-1278): the
 * same grouped GEMM over device arrays of device pointers, one entry per group: packed rows and their 128 x 4 scale tiles,
 * packed weights [m][k / 2] and their scale tiles, bf16 output [rows of the group][m], a pointer to the group's alpha, and
 * the row count of every group (at most max_n).  In front of the GEMM a small kernel patches one tensor map per group and
 * operand from the tables (tensormap.replace), so nothing is read back to the host and the call can be captured. */
EIDER_B200_API int infer_cutlass_fp4_grouped_gemm_supported(uint32_t m, uint32_t max_n, uint32_t k, uint32_t groups);
EIDER_B200_API void* infer_cutlass_fp4_grouped_gemm_create(uint32_t m, uint32_t max_n, uint32_t k, uint32_t groups);
EIDER_B200_API void infer_cutlass_fp4_grouped_gemm_destroy(void* plan);
EIDER_B200_API cudaError_t infer_cutlass_fp4_grouped_gemm_on_stream(void* plan, const uint8_t* const* a_values,
                                                                    const uint8_t* const* a_scales,
                                                                    const uint8_t* const* b_values,
                                                                    const uint8_t* const* b_scales, uint16_t* const* output,
                                                                    float* const* alpha, const uint32_t* tokens_per_expert,
                                                                    cudaStream_t stream);
EIDER_B200_API cudaError_t eider_b200_grouped_plan_status(void* plan, uint32_t* host_status);
/* crates/eider-cuda/src/ffi.rs:1931 (kernel non_gemm.cu:3735-3780): un-permute + weighted sum, f32 [rows][len]. */
EIDER_B200_API cudaError_t infer_moe_weighted_accumulate_sorted_bf16_batch_on_stream(
    const uint32_t* route_to_sorted, const float* route_weights, const uint16_t* sorted_inputs, float* output, uint32_t rows,
    uint32_t len, uint32_t routes_per_row, cudaStream_t stream);

/* Tile-shape override (64, 128, 192 or 256 weight rows per tile; 512 = 256 x 256 tiles computed by pairs of CTAs
 * with tcgen05 cta_group::2, 384 = 256 x 192 tiles on such pairs) and the kernel status word of a plan
 * (0 = ok; non-zero = a bounded device wait expired, low byte = which). */
EIDER_B200_API int eider_b200_gemm_plan_set_block_n(void* plan, uint32_t block_n);
EIDER_B200_API uint32_t eider_b200_gemm_plan_block_n(void* plan); /* the tile code in use (0 for a null plan) */
/* Split K of a dense plan (no reference counterpart; the reference's cuBLASLt heuristics choose theirs).  A shape with few
 * output tiles and a long K (a 128..512-token chunk through a down projection) leaves most SMs idle while a few stream the
 * whole K; with `splits` > 1 every tile's K range is divided over that many work items, which write fp32 partial sums into
 * a workspace the plan owns (splits x tokens x out_features floats, allocated by this call or at creation), and a dependent
 * launch sums them in split order and applies alpha, the scales, beta * C and the output conversion exactly as the
 * unsplit epilogue does.  Plans choose a split count themselves at creation and when the tile shape is set; this call
 * overrides it (1 = off; at most 16; cudaErrorInvalidValue when a split would be empty).  Ignored while the fused
 * all-gather is on. */
EIDER_B200_API cudaError_t eider_b200_gemm_plan_set_k_splits(void* plan, uint32_t splits);
EIDER_B200_API uint32_t eider_b200_gemm_plan_k_splits(void* plan); /* the split count in use (0 for a null plan) */
/* The choices a dense plan makes at creation, as plain functions of the shape and the device's SM count (no device is
 * touched): the tile code for m tokens x n output features, and the K split count for that tile code (is_nvfp4: 1 for
 * NVFP4 operands, 0 for FP8).  0 for a zero extent or fewer than two SMs. */
EIDER_B200_API uint32_t eider_b200_gemm_pick_tile(uint32_t m, uint32_t n, uint32_t sms);
EIDER_B200_API uint32_t eider_b200_gemm_pick_k_splits(int is_nvfp4, uint32_t m, uint32_t n, uint32_t k, uint32_t block_n, uint32_t sms);
/* Fused all-gather for a column-sharded dense layer (no reference counterpart: the reference is single-GPU).  peers[q]
 * points at this rank's first output column inside rank q's full [tokens][ld_out] output (its own buffer included),
 * mapped into this process (CUDA IPC / symmetric memory), 32-byte aligned; count <= 8.  While set, the GEMM's epilogue
 * writes every output tile to all of them with plain stores over NVLink and the `d` argument of the run call is ignored;
 * beta must be 0.  The caller still has to synchronise the ranks before the outputs are read or overwritten.  count = 0
 * switches it off. */
EIDER_B200_API cudaError_t eider_b200_gemm_plan_set_output_peers(void* plan, void* const* peers, uint32_t count,
                                                                 uint32_t ld_out);
/* Optional on top of set_output_peers: `multicast_block` = the same column block as an address inside an NVLink multicast
 * mapping that covers every rank's output (CUDA multicast object / symmetric memory's multicast pointer), 16-byte
 * aligned.  The CTA-pair kernel then writes every output tile once with multimem.st and the switch copies it to all
 * ranks, so a tile leaves the GPU once instead of once per peer; other kernels and outputs keep using the peer list.
 * NULL switches it off.  No reference counterpart. */
EIDER_B200_API cudaError_t eider_b200_gemm_plan_set_output_multicast(void* plan, void* multicast_block);
EIDER_B200_API cudaError_t eider_b200_gemm_plan_status(void* plan, uint32_t* host_status);

/* ---- meeting of the ranks of one node (no reference counterpart: the reference is single-GPU) --------- */

/* Bounded device-side barrier over peer memory, for the step of the fused all-gather where every rank's columns must have
 * arrived.  signal_pads[q] = rank q's pad of eider_b200_peer_barrier_pad_bytes() zeroed bytes in memory every rank can
 * write (symmetric memory / CUDA IPC), `state` = eider_b200_peer_barrier_state_bytes() zeroed bytes of this rank's own
 * device memory (16 per-channel epochs, then one status word).  All ranks must call with the same channel in the same
 * order.  The wait gives up after timeout_cycles SM cycles (0 = about one second), records 0xBA000000 | channel << 8 |
 * missing rank in the status word and returns: nothing spins forever and the context stays usable. */
EIDER_B200_API size_t eider_b200_peer_barrier_pad_bytes(void);
EIDER_B200_API size_t eider_b200_peer_barrier_state_bytes(void);
EIDER_B200_API cudaError_t eider_b200_peer_barrier_on_stream(void* const* signal_pads, uint32_t world, uint32_t rank,
                                                             uint32_t channel, uint32_t* state, uint64_t timeout_cycles,
                                                             cudaStream_t stream);

/* ---- decode-side routed MoE and lm-head arg-max (CUDA cores, device pointer tables) ----------------------------- */

/* crates/eider-cuda/src/ffi.rs:3320 and :3348 (kernels non_gemm.cu:13316-13397): slot g multiplies the weights of expert
 * indices[g] (table entries: packed [out][in/2], row-major scales [out][in/16], weight_scale_2) with the shared f32 input
 * (or with input_table[g]) and writes output_table[g][out].  Slots whose expert is >= table_len are skipped, as in the
 * reference.  This implementation needs in_features % 32 == 0 and 16-byte aligned weight rows. */
EIDER_B200_API cudaError_t infer_nvfp4_w4a16_grouped_matvec_f32_on_stream(
    const uint32_t* indices, const float* input, const uint8_t* const* packed_weight_table, const uint8_t* const* weight_scale_table,
    const float* weight_scale_2_table, float* const* output_table, uint32_t table_len, uint32_t groups, uint32_t out_features,
    uint32_t in_features, cudaStream_t stream);
EIDER_B200_API cudaError_t infer_nvfp4_w4a16_grouped_inputs_matvec_f32_on_stream(
    const uint32_t* indices, const float* const* input_table, const uint8_t* const* packed_weight_table,
    const uint8_t* const* weight_scale_table, const float* weight_scale_2_table, float* const* output_table, uint32_t table_len,
    uint32_t groups, uint32_t out_features, uint32_t in_features, cudaStream_t stream);
/* crates/eider-cuda/src/ffi.rs:3333 (kernel non_gemm.cu:13640-13724): routes sorted by expert; route r of the sorted order
 * multiplies inputs[sorted_routes[r]] by the matrix of expert sorted_experts[r] into outputs[sorted_routes[r]], times
 * globals[expert].  in_features % 32 == 0 here (the reference: % 16, at most 3072); `offsets` must be non-null and is not read. */
EIDER_B200_API cudaError_t infer_nvfp4_w4a16_reuse_matvec_f32_on_stream(const uint32_t* sorted_routes,
                                                                        const uint32_t* sorted_experts, const uint32_t* offsets,
                                                                        const float* const* inputs, const uint8_t* const* weights,
                                                                        const uint8_t* const* scales, const float* globals,
                                                                        float* const* outputs, uint32_t routes, uint32_t experts,
                                                                        uint32_t out_features, uint32_t in_features,
                                                                        cudaStream_t stream);
/* crates/eider-cuda/src/ffi.rs:589-642 (crates/eider-cuda/native/cutlass_gemv.cu:277-880): grouped W4A4 GEMV with F32 output;
 * a = expert weights with tiled scales (found through tables), b = one NVFP4 activation row with tiled scales (outer = 0).
 * indexed_a: d[g] = alpha * A[indices[g]] . b; ..._tiled_scales: per-expert alpha_table, c is not read (beta 0);
 * contiguous_b: group g uses table entry g and writes d + g * m.  The plan records the shape only. */
EIDER_B200_API int infer_cutlass_fp4_grouped_gemv_f32_supported(uint32_t m, uint32_t k, uint32_t groups);
EIDER_B200_API void* infer_cutlass_fp4_grouped_gemv_f32_create(uint32_t m, uint32_t k, uint32_t groups);
EIDER_B200_API void infer_cutlass_fp4_grouped_gemv_f32_destroy(void* plan);
EIDER_B200_API cudaError_t infer_cutlass_fp4_grouped_gemv_f32_indexed_a_on_stream(
    void* plan, const uint32_t* indices, const uint8_t* const* a_values_table, const uint8_t* const* a_scales_table, uint32_t table_len,
    const uint8_t* b_values, const uint8_t* b_scales, float* const* d, float alpha, cudaStream_t stream);
EIDER_B200_API cudaError_t infer_cutlass_fp4_grouped_gemv_f32_indexed_a_tiled_scales_on_stream(
    void* plan, const uint32_t* indices, const uint8_t* const* a_values_table, const uint8_t* const* a_scales_table,
    const float* alpha_table, uint32_t table_len, const uint8_t* b_values, const uint8_t* b_scales, const float* c, float* const* d,
    cudaStream_t stream);
EIDER_B200_API cudaError_t infer_cutlass_fp4_grouped_gemv_f32_contiguous_b_on_stream(
    void* plan, const uint8_t* const* a_values_table, const uint8_t* const* a_scales_table, const uint8_t* b_values,
    const uint8_t* b_scales, float* d, float alpha, cudaStream_t stream);
/* crates/eider-cuda/src/ffi.rs:1887 and kernel non_gemm.cu:3558-3593: per slot, g = gate * alpha[expert], u = up * alpha[expert],
 * value = g * sigmoid(g) * u; f32 out, or value / input_scale[expert] -> NVFP4 with one scale byte per 16 values in plain
 * order (a slot whose input scale is not positive and finite is left untouched, as in the reference). */
EIDER_B200_API cudaError_t infer_moe_silu_slots_f32_on_stream(const uint32_t* indices, const float* const* gate_up_table,
                                                              float* const* output_table, const float* gate_up_alpha_table,
                                                              uint32_t rows, uint32_t groups, cudaStream_t stream);
EIDER_B200_API cudaError_t infer_moe_silu_quantize_slots_nvfp4_simple_scales_on_stream(
    const uint32_t* indices, const float* const* gate_up_table, uint8_t* const* packed_table, uint8_t* const* scales_table,
    const float* input_scale_table, const float* gate_up_alpha_table, uint32_t rows, uint32_t groups, cudaStream_t stream);
/* crates/eider-cuda/src/ffi.rs:1898 and :1908 (kernels non_gemm.cu:3595-3639): output[row][c] = sum over the row's slots of
 * inputs[route][c] * route_weights[route] * alpha_table[indices[route]], slot order. */
EIDER_B200_API cudaError_t infer_moe_weighted_accumulate_slots_f32_on_stream(const uint32_t* indices, const float* route_weights,
                                                                             const float* const* inputs, const float* alpha_table,
                                                                             float* output, uint32_t len, uint32_t groups,
                                                                             cudaStream_t stream);
EIDER_B200_API cudaError_t infer_moe_weighted_accumulate_slots_f32_batch_on_stream(const uint32_t* indices, const float* route_weights,
                                                                                   const float* const* inputs, const float* alpha_table,
                                                                                   float* output, uint32_t rows, uint32_t len,
                                                                                   uint32_t groups, cudaStream_t stream);
/* Kernels non_gemm.cu:3823-3875: the same sum + shared_output * sigmoid(shared_gate_logit[row]) + residual, rounded to bf16
 * precision (the value stays f32). */
EIDER_B200_API cudaError_t infer_qwen36_ffn_finalize_routed_f32_on_stream(
    const uint32_t* indices, const float* route_weights, const float* const* routed_outputs, const float* alpha_table,
    const float* shared_gate_logit, const float* shared_output, const float* residual, float* output, uint32_t len, uint32_t groups,
    cudaStream_t stream);
EIDER_B200_API cudaError_t infer_qwen36_ffn_finalize_routed_batch_f32_on_stream(
    const uint32_t* indices, const float* route_weights, const float* const* routed_outputs, const float* alpha_table,
    const float* shared_gate_logit, const float* shared_output, const float* residual, float* output, uint32_t rows, uint32_t cols,
    uint32_t groups_per_row, cudaStream_t stream);
/* crates/eider-cuda/src/ffi.rs:3473 (kernels non_gemm.cu:13423-13482, 8287-8328): arg-max of weight_scale_2 * W . x over the
 * output features without materialising the logits; ties go to the lower row.  scratch_value / scratch_index: scratch_len
 * entries each (any scratch_len >= 1; up to 1024 are used).  warps_per_block must be 4, 8, 16 or 32 as in the reference and
 * has no other meaning here; in_features % 32 == 0. */
EIDER_B200_API cudaError_t infer_nvfp4_w4a16_top1_f32_on_stream(const float* input, const uint8_t* packed_weight,
                                                                const uint8_t* weight_scale, float* scratch_value,
                                                                uint32_t* scratch_index, uint32_t scratch_len, uint32_t* out_index,
                                                                float* out_value, uint32_t out_features, uint32_t in_features,
                                                                float weight_scale_2, uint32_t warps_per_block, cudaStream_t stream);

/* ---- host-side weight ingest (no device work; host pointers) ------------------------------------------------- */
/* Return codes of this group: 0 ok, 1 shape error, 2 format error, 3 I/O error (the reference's Error::Shape /
 * Error::Format kinds, crates/eider-format/src/lib.rs).
 *
 * Nvfp4Artifact, the reference's per-linear disk record, bit-compatible in both directions
 * (crates/eider-format/src/nvfp4_artifact.rs:12-75: "EIDNVF4\0", version 1, 60-byte little-endian header, prefix, packed
 * E2M1 bytes [out][in/2], E4M3 K16 scales [out][in/16]); written through a temporary file and a rename. */
EIDER_B200_API int eider_b200_nvfp4_artifact_write(const char* path, const char* prefix, uint64_t out_features,
                                                   uint64_t in_features, const uint8_t* packed_weight, uint64_t packed_len,
                                                   const uint8_t* weight_scale, uint64_t scale_len, float weight_scale_2,
                                                   float input_scale);
EIDER_B200_API int eider_b200_nvfp4_artifact_read_header(const char* path, uint64_t* out_features, uint64_t* in_features,
                                                         uint64_t* packed_len, uint64_t* scale_len, uint64_t* prefix_len,
                                                         float* weight_scale_2, float* input_scale);
EIDER_B200_API int eider_b200_nvfp4_artifact_read(const char* path, char* prefix, uint64_t prefix_capacity,
                                                  uint8_t* packed_weight, uint64_t packed_capacity, uint8_t* weight_scale,
                                                  uint64_t scale_capacity);
/* compressed-tensors stores divisors: weight_scale_2 = 1 / weight_global_scale, input_scale = 1 / input_global_scale
 * (crates/eider-format/src/modelopt.rs:480-519, 1137-1145); non-positive or non-finite divisors are format errors. */
EIDER_B200_API int eider_b200_compressed_tensors_globals(float weight_global_scale, float input_global_scale,
                                                         float* weight_scale_2, float* input_scale);
/* MXFP4 -> NVFP4 scale widening (crates/eider-format/src/modelopt.rs:173-248): `count` E8M0 K32 scales become 2 * count
 * UE4M3 K16 scales; a NaN code or a power of two UE4M3 cannot hold exactly is a format error. */
EIDER_B200_API int eider_b200_mxfp4_scales_to_nvfp4(const uint8_t* e8m0_scales, uint64_t count, uint8_t* ue4m3_scales);
/* GGML NVFP4 blocks (four scales + 32 split-half nibble bytes per 64 values) -> ModelOpt row-major storage, no decoding
 * (crates/eider-format/src/gguf_nvfp4.rs:12-64). */
EIDER_B200_API int eider_b200_gguf_nvfp4_unpack(const uint8_t* blocks, uint64_t bytes, uint64_t out_features,
                                                uint64_t in_features, float global_scale, uint8_t* packed_weight,
                                                uint8_t* weight_scale);
/* ModelOptNvfp4Linear::quantize_values and its front ends (crates/eider-format/src/modelopt.rs:524-716), unit global scale.
 * source_kind 0: f32 values; 1: bf16 bits; 2: FP8 E4M3 bytes times channel_scale[row] (or tensor_scale when NULL);
 * 3: FP8 E4M3 bytes times 128 x 128 E8M0 block scales. */
EIDER_B200_API int eider_b200_nvfp4_requantize_host(int source_kind, const void* values, const float* channel_scale,
                                                    float tensor_scale, const uint8_t* block_scale_e8m0, uint64_t out_features,
                                                    uint64_t in_features, uint8_t* packed_weight, uint8_t* weight_scale);
/* modelopt_scales_to_cublaslt on the host (crates/eider-format/src/modelopt.rs:1148-1161). */
EIDER_B200_API void eider_b200_nvfp4_scales_to_tiled_host(const uint8_t* scales_row_major, uint8_t* scales_tiled,
                                                          uint64_t out_features, uint64_t in_features);
/* Prepared-layout cache "EIDB2P01" (48-byte header: magic, version 1, out, in, weight bytes, scale bytes, weight_scale_2;
 * then the packed bytes as they are and the 128 x 4 tiled scales), the analogue of the reference's EIDW4A01 file
 * (crates/eider-cuda/src/kernels/sm121_w4a16.rs:18-20, 146-240).  `matches` returns 1 when the file holds the complete
 * payload for the shape. */
EIDER_B200_API int eider_b200_prepared_cache_write(const char* path, uint64_t out_features, uint64_t in_features,
                                                   const uint8_t* packed_weight, const uint8_t* scales_tiled,
                                                   float weight_scale_2);
EIDER_B200_API int eider_b200_prepared_cache_matches(const char* path, uint64_t out_features, uint64_t in_features);
EIDER_B200_API int eider_b200_prepared_cache_read(const char* path, uint64_t out_features, uint64_t in_features,
                                                  uint8_t* packed_weight, uint8_t* scales_tiled, float* weight_scale_2);

/* ---- expert-parallel routed MoE over peer memory (no reference counterpart) ------------------------------ */

/* Experts are split evenly over `world` ranks of one node, tokens start sharded by rows.  Routes travel by plain peer stores
 * into receive buffers every rank keeps in peer-writable memory; all counts stay on the device (nothing is read back, the
 * whole step can be captured in a graph).  Order per step, with a barrier (above) between the numbered groups:
 *   1. top-k and route sort by global expert on the local tokens, then eider_b200_ep_publish_counts_on_stream;
 *   2. eider_b200_ep_offsets_on_stream, the activation quantizer on the local tokens (unit global scale), then
 *      eider_b200_ep_dispatch_rows_on_stream;
 *   3. eider_b200_ep_expand_experts_on_stream, the grouped GEMMs and the SiLU quantizer (..._limited_...) on the received
 *      rows with recv_offsets as expert offsets, then eider_b200_ep_return_rows_on_stream;
 *   4. infer_moe_weighted_accumulate_sorted_bf16_batch_on_stream on the return buffer with the identity route map.
 * Every pointer table has `world` entries, entry q = rank q's buffer mapped into this process (its own included).
 * counts_all[q]: uint32 [world][experts].  recv_packed[q]: capacity x in_features / 2 bytes; recv_scales[q]:
 * (ceil(capacity / 128) + experts / world) scale tiles; recv_origin[q]: uint32 [capacity]; return_rows[q]: bf16
 * [routes of rank q][out_features].  capacity >= the most rows a rank can receive (all routes of all ranks is always safe);
 * routes per rank < 2^24; in_features % 32 == 0; out_features % 8 == 0. */
EIDER_B200_API cudaError_t eider_b200_ep_publish_counts_on_stream(const uint32_t* expert_counts, void* const* counts_all,
                                                                  uint32_t world, uint32_t rank, uint32_t experts,
                                                                  cudaStream_t stream);
/* expert_base[e] = first row of expert e in its owner's receive buffer, before_me[e] = rows of e from lower ranks,
 * recv_offsets[experts / world + 1] = this rank's expert offsets over what it receives, recv_total[1] = their sum. */
EIDER_B200_API cudaError_t eider_b200_ep_offsets_on_stream(const uint32_t* counts_all, uint32_t world, uint32_t rank,
                                                           uint32_t experts, uint32_t* expert_base, uint32_t* before_me,
                                                           uint32_t* recv_offsets, uint32_t* recv_total, cudaStream_t stream);
/* source_packed / source_scales: the local tokens quantized once (tiled scales, outer = token); sorted_routes /
 * sorted_experts / local_offsets: the local route sort by global expert. */
EIDER_B200_API cudaError_t eider_b200_ep_dispatch_rows_on_stream(
    const uint8_t* source_packed, const uint8_t* source_scales, const uint32_t* sorted_routes, const uint32_t* sorted_experts,
    const uint32_t* local_offsets, const uint32_t* expert_base, const uint32_t* before_me, void* const* recv_packed,
    void* const* recv_scales, void* const* recv_origin, uint32_t routes, uint32_t routes_per_row, uint32_t in_features,
    uint32_t scale_tile_bytes, uint32_t experts, uint32_t world, uint32_t rank, cudaStream_t stream);
/* sorted_experts[row] for received rows: the local expert whose range holds the row (experts / world past the total). */
EIDER_B200_API cudaError_t eider_b200_ep_expand_experts_on_stream(const uint32_t* recv_offsets, uint32_t local_experts,
                                                                  uint32_t* sorted_experts, uint32_t capacity,
                                                                  cudaStream_t stream);
/* rows [capacity][out_features] bf16: row i < *recv_total goes to return_rows[source rank of i] at the route's own index. */
EIDER_B200_API cudaError_t eider_b200_ep_return_rows_on_stream(const uint16_t* rows, const uint32_t* recv_origin,
                                                               const uint32_t* recv_total, void* const* return_rows,
                                                               uint32_t capacity, uint32_t out_features, uint32_t world,
                                                               cudaStream_t stream);

#ifdef __cplusplus
}
#endif

#endif /* EIDER_B200_H */
