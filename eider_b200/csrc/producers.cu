// Producers in front of the NVFP4 quantizer, fused and staged.
//
// The reference fuses the operator that produces an activation with the quantizer that feeds the next GEMM
// (crates/eider-cuda/native/non_gemm.cu:421-557, 8951-9060, 12029-12120) and keeps the unfused kernels as the staged
// path its tests compare with, byte for byte.  This file holds both halves for the element-wise producers:
//   staged:  RMSNorm, RMSNorm + residual, SiLU(gate) * up, GELU-tanh(gate) * up, head unpack, gated RMSNorm  -> f32
//   fused:   GELU-tanh * up -> NVFP4, head unpack -> NVFP4 (f32 / bf16 input), gated RMSNorm -> NVFP4,
//            vector quantizer with linear ("simple") scales
// plus the two in-place channel scalings of the FP8 path.  Every formula and every sum comes from rowops.cuh, which the
// fused RMSNorm producers in quantize.cu use too, so fused == staged holds by construction.
//
// HBM-bound element-wise work: one thread per 16-element block on the quantizing kernels (128-bit loads, one 64-bit
// packed store, one scale byte), one thread per element or per four elements on the staged ones.
#include "common.cuh"
#include "rowops.cuh"
#include "eider_b200.h"

namespace eider {
namespace {

bool bad_scale(float s) { return !(s > 0.0f) || !isfinite(s); }

bool aligned16(const void* a, const void* b = nullptr, const void* c = nullptr, const void* d = nullptr) {
    return ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(c) |
             reinterpret_cast<uintptr_t>(d)) & 15) == 0;
}

// ---- staged kernels ---------------------------------------------------------------------------------------

// RMSNorm (non_gemm.cu:631-667) and RMSNorm + residual (non_gemm.cu:700-727), one CTA of 256 threads per row.
template <bool ADD, bool VEC>
__global__ void __launch_bounds__(256) rms_norm_f32_kernel(const float* __restrict__ input, const float* __restrict__ weight,
                                                           const float* __restrict__ residual, float* __restrict__ output,
                                                           uint32_t cols, float eps) {
    __shared__ float red[8];
    const size_t off = static_cast<size_t>(blockIdx.x) * cols;
    const float ss = VEC ? rowops::thread_sum_squares_f4(input + off, cols) : rowops::thread_sum_squares_scalar(input + off, cols);
    const float inv = rowops::inverse_rms(rowops::block_sum_ordered(ss, red), cols, eps);
    if (VEC) {
        for (uint32_t i = threadIdx.x; i < cols / 4; i += blockDim.x) {
            const float4 v = __ldg(reinterpret_cast<const float4*>(input + off) + i);
            const float4 w = __ldg(reinterpret_cast<const float4*>(weight) + i);
            float4 h;
            if (ADD) {
                const float4 r = __ldg(reinterpret_cast<const float4*>(residual + off) + i);
                h.x = rowops::normed_add(v.x, inv, w.x, r.x);
                h.y = rowops::normed_add(v.y, inv, w.y, r.y);
                h.z = rowops::normed_add(v.z, inv, w.z, r.z);
                h.w = rowops::normed_add(v.w, inv, w.w, r.w);
            } else {
                h.x = rowops::normed(v.x, inv, w.x);
                h.y = rowops::normed(v.y, inv, w.y);
                h.z = rowops::normed(v.z, inv, w.z);
                h.w = rowops::normed(v.w, inv, w.w);
            }
            reinterpret_cast<float4*>(output + off)[i] = h;
        }
    } else {
        for (uint32_t i = threadIdx.x; i < cols; i += blockDim.x) {
            const float v = __ldg(input + off + i), w = __ldg(weight + i);
            output[off + i] = ADD ? rowops::normed_add(v, inv, w, __ldg(residual + off + i)) : rowops::normed(v, inv, w);
        }
    }
}

// Gated RMSNorm (non_gemm.cu:11514-11549): x * inverse_rms * weight * silu(gate), one CTA per row.
__global__ void __launch_bounds__(256) gated_rms_norm_f32_kernel(const float* __restrict__ input, const float* __restrict__ gate,
                                                                 const float* __restrict__ weight, float* __restrict__ output,
                                                                 uint32_t cols, float eps) {
    __shared__ float red[8];
    const size_t off = static_cast<size_t>(blockIdx.x) * cols;
    const float inv = rowops::inverse_rms(rowops::block_sum_ordered(rowops::thread_sum_squares_scalar(input + off, cols), red), cols, eps);
    for (uint32_t i = threadIdx.x; i < cols; i += blockDim.x) {
        const float g = __ldg(gate + off + i);
        const float silu = __fdiv_rn(g, __fadd_rn(1.0f, expf(-g)));
        output[off + i] = __fmul_rn(rowops::normed(__ldg(input + off + i), inv, __ldg(weight + i)), silu);
    }
}

enum Act { kSiluHalves = 0, kGeluPair = 1 };

// Activation(gate) * up -> f32.  kSiluHalves: rows of [gate | up] (non_gemm.cu:1357-1370); kGeluPair: separate gate and
// up arrays of `len` elements (non_gemm.cu:1226-1246), cols = len and rows = 1.
template <int ACT>
__global__ void __launch_bounds__(256) act_mul_f32_kernel(const float* __restrict__ gate, const float* __restrict__ up,
                                                          float* __restrict__ output, uint32_t rows, uint32_t cols, float limit) {
    const size_t idx = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= static_cast<size_t>(rows) * cols) return;
    if (ACT == kSiluHalves) {
        const size_t row = idx / cols, col = idx - row * cols;
        const size_t base = row * cols * 2;
        float g = __ldg(gate + base + col), u = __ldg(gate + base + cols + col);
        if (limit > 0.0f) {  // clamped form (non_gemm.cu:1328-1338): gate from above, up from both sides
            g = fminf(g, limit);
            u = fminf(fmaxf(u, -limit), limit);
        }
        output[idx] = rowops::silu_div_mul(g, u);
    } else {
        output[idx] = rowops::gelu_tanh_mul(__ldg(gate + idx), __ldg(up + idx));
    }
}

// Attention output [heads][tokens][head_dim] -> token-major rows starting at output_row_offset (non_gemm.cu:8898-8915).
__global__ void __launch_bounds__(256) unpack_heads_f32_kernel(const float* __restrict__ input, float* __restrict__ output,
                                                               uint32_t tokens, uint32_t heads, uint32_t head_dim,
                                                               uint32_t output_row_offset) {
    const size_t index = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    const size_t total = static_cast<size_t>(tokens) * heads * head_dim;
    if (index >= total) return;
    const uint32_t dim = static_cast<uint32_t>(index % head_dim);
    const uint32_t head = static_cast<uint32_t>((index / head_dim) % heads);
    const uint32_t token = static_cast<uint32_t>(index / (static_cast<size_t>(heads) * head_dim));
    output[((static_cast<size_t>(output_row_offset) + token) * heads + head) * head_dim + dim] =
        __ldg(input + (static_cast<size_t>(head) * tokens + token) * head_dim + dim);
}

// values[r][c] *= channel_scale[c] * row_scale[r] (non_gemm.cu: infer_scale_channel_f32_device_row_scalar_kernel);
// rows == 0 selects the one-scalar form, values[i] *= channel_scale[i] * scalar[0].
__global__ void __launch_bounds__(256) scale_channel_kernel(float* __restrict__ values, const float* __restrict__ channel_scale,
                                                            const float* __restrict__ row_scale, uint32_t channels, size_t len,
                                                            int per_row) {
    const size_t idx = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= len) return;
    const float s = per_row ? __fmul_rn(__ldg(channel_scale + idx % channels), __ldg(row_scale + idx / channels))
                            : __fmul_rn(__ldg(channel_scale + idx), __ldg(row_scale));
    values[idx] = __fmul_rn(values[idx], s);
}

// ---- fused quantizing producers -----------------------------------------------------------------------------

// Store one quantized block of a row whose length is a multiple of 16.
__device__ __forceinline__ void store_block(uint8_t* packed, uint8_t* scales, uint32_t row, uint32_t b, uint32_t cols,
                                            const float (&v)[16]) {
    uint2 bytes;
    const uint8_t sc = quantize_block16(v, 16, &bytes);
    *reinterpret_cast<uint2*>(packed + static_cast<size_t>(row) * (cols / 2) + b * 8) = bytes;
    scales[tiled_scale_offset(row, b, cols)] = sc;
}

// GELU-tanh(gate) * up / input_scale -> NVFP4 (non_gemm.cu:421-486).  grid = (ceil(blocks / 256), rows).
__global__ void __launch_bounds__(256) gelu_mul_quantize_kernel(const float* __restrict__ gate, const float* __restrict__ up,
                                                                uint8_t* __restrict__ packed, uint8_t* __restrict__ scales,
                                                                uint32_t cols, float input_scale) {
    const uint32_t row = blockIdx.y;
    const uint32_t b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= cols / 16) return;
    const size_t base = static_cast<size_t>(row) * cols + b * 16;
    const Divisor di = make_divisor(input_scale);
    float v[16];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        const float4 g4 = __ldg(reinterpret_cast<const float4*>(gate + base) + q);
        const float4 u4 = __ldg(reinterpret_cast<const float4*>(up + base) + q);
        v[4 * q + 0] = div_rn(rowops::gelu_tanh_mul(g4.x, u4.x), di);
        v[4 * q + 1] = div_rn(rowops::gelu_tanh_mul(g4.y, u4.y), di);
        v[4 * q + 2] = div_rn(rowops::gelu_tanh_mul(g4.z, u4.z), di);
        v[4 * q + 3] = div_rn(rowops::gelu_tanh_mul(g4.w, u4.w), di);
    }
    store_block(packed, scales, row, b, cols, v);
}

template <typename T> struct LoadOne;
template <> struct LoadOne<float> {
    static __device__ __forceinline__ float at(const float* p, size_t i) { return __ldg(p + i); }
};
template <> struct LoadOne<uint16_t> {
    static __device__ __forceinline__ float at(const uint16_t* p, size_t i) { return bf16_bits_to_float(__ldg(p + i)); }
};

// Attention output [heads][tokens][head_dim] -> NVFP4 rows [output_row_offset + token][heads * head_dim]
// (non_gemm.cu:8951-9017).  A 16-element block never straddles two heads when head_dim % 16 == 0 (checked on the host),
// so each thread reads 16 consecutive source elements.  grid = (ceil(blocks / 128), tokens).
template <typename T>
__global__ void __launch_bounds__(128) unpack_heads_quantize_kernel(const T* __restrict__ input, uint8_t* __restrict__ packed,
                                                                    uint8_t* __restrict__ scales, uint32_t tokens, uint32_t heads,
                                                                    uint32_t head_dim, uint32_t output_row_offset,
                                                                    float input_scale) {
    const uint32_t token = blockIdx.y;
    const uint32_t features = heads * head_dim;
    const uint32_t b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= features / 16) return;
    const uint32_t head = (b * 16) / head_dim, dim = (b * 16) % head_dim;
    const size_t src = (static_cast<size_t>(head) * tokens + token) * head_dim + dim;
    const Divisor di = make_divisor(input_scale);
    float v[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = div_rn(LoadOne<T>::at(input, src + i), di);
    store_block(packed, scales, output_row_offset + token, b, features, v);
}

// Per-head gated RMSNorm -> NVFP4 for head_dim = 128 (non_gemm.cu:12029-12094): one CTA of 128 threads per (row, head);
// value = x * inverse_rms * weight * silu(gate) / input_scale; threads 0..7 then quantize the head's eight blocks out
// of shared memory.
__global__ void __launch_bounds__(128) gated_rms_norm_quantize_kernel(const float* __restrict__ input, const float* __restrict__ gate,
                                                                      const float* __restrict__ weight, uint8_t* __restrict__ packed,
                                                                      uint8_t* __restrict__ scales, uint32_t heads, float eps,
                                                                      float input_scale) {
    __shared__ float red[4];
    __shared__ float staged[128];
    const uint32_t row = blockIdx.x / heads, head = blockIdx.x % heads;
    const uint32_t cols = heads * 128;
    const size_t off = static_cast<size_t>(row) * cols + head * 128;
    const float x = __ldg(input + off + threadIdx.x);
    const float inv = rowops::inverse_rms(rowops::block_sum_ordered(fmaf(x, x, 0.0f), red), 128, eps);
    const float g = __ldg(gate + off + threadIdx.x);
    const float silu = __fdiv_rn(g, __fadd_rn(1.0f, expf(-g)));
    const Divisor di = make_divisor(input_scale);
    staged[threadIdx.x] = div_rn(__fmul_rn(rowops::normed(x, inv, __ldg(weight + threadIdx.x)), silu), di);
    __syncthreads();
    if (threadIdx.x < 8) {
        float v[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) v[i] = staged[threadIdx.x * 16 + i];
        store_block(packed, scales, row, head * 8 + threadIdx.x, cols, v);
    }
}

// One vector of `rows` values with one scale byte per 16 values in plain order (non_gemm.cu:510-541).
__global__ void __launch_bounds__(128) quantize_vector_simple_scales_kernel(const float* __restrict__ input, uint8_t* __restrict__ packed,
                                                                            uint8_t* __restrict__ scales, uint32_t rows,
                                                                            float input_scale) {
    const uint32_t b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= (rows + 15) / 16) return;
    const uint32_t valid = min(16u, rows - b * 16);
    const Divisor di = make_divisor(input_scale);
    float v[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = static_cast<uint32_t>(i) < valid ? div_rn(__ldg(input + b * 16 + i), di) : 0.0f;
    uint2 bytes;
    scales[b] = quantize_block16(v, valid, &bytes);
    const uint32_t w[2] = {bytes.x, bytes.y};
    for (uint32_t i = 0; i < (valid + 1) / 2; ++i) packed[b * 8 + i] = static_cast<uint8_t>(w[i / 4] >> ((i % 4) * 8));
}

}  // namespace
}  // namespace eider

using namespace eider;

extern "C" {

cudaError_t infer_rms_norm_f32_on_stream(const float* input, const float* weight, float* output, uint32_t rows, uint32_t cols,
                                         float eps, cudaStream_t stream) {
    if (!input || !weight || !output || rows == 0 || cols == 0) return cudaErrorInvalidValue;
    if (cols % 4 == 0 && aligned16(input, weight, output))
        rms_norm_f32_kernel<false, true><<<rows, 256, 0, stream>>>(input, weight, nullptr, output, cols, eps);
    else
        rms_norm_f32_kernel<false, false><<<rows, 256, 0, stream>>>(input, weight, nullptr, output, cols, eps);
    return cudaGetLastError();
}

cudaError_t infer_rms_norm_add_f32_on_stream(const float* input, const float* weight, const float* residual, float* output,
                                             uint32_t rows, uint32_t cols, float eps, cudaStream_t stream) {
    if (!input || !weight || !residual || !output || rows == 0 || cols == 0 || eps < 0.0f || !isfinite(eps))
        return cudaErrorInvalidValue;
    if (cols % 4 == 0 && aligned16(input, weight, residual, output))
        rms_norm_f32_kernel<true, true><<<rows, 256, 0, stream>>>(input, weight, residual, output, cols, eps);
    else
        rms_norm_f32_kernel<true, false><<<rows, 256, 0, stream>>>(input, weight, residual, output, cols, eps);
    return cudaGetLastError();
}

cudaError_t infer_gated_rms_norm_f32_on_stream(const float* input, const float* gate, const float* weight, float* output,
                                               uint32_t rows, uint32_t cols, float eps, cudaStream_t stream) {
    if (!input || !gate || !weight || !output || rows == 0 || cols == 0) return cudaErrorInvalidValue;
    gated_rms_norm_f32_kernel<<<rows, 256, 0, stream>>>(input, gate, weight, output, cols, eps);
    return cudaGetLastError();
}

cudaError_t infer_silu_mul_halves_f32_batch_on_stream(const float* gate_up, float* output, uint32_t rows, uint32_t cols,
                                                      cudaStream_t stream) {
    if (!gate_up || !output || rows == 0 || cols == 0) return cudaErrorInvalidValue;
    const size_t len = static_cast<size_t>(rows) * cols;
    act_mul_f32_kernel<kSiluHalves><<<static_cast<uint32_t>((len + 255) / 256), 256, 0, stream>>>(gate_up, nullptr, output, rows, cols, 0.0f);
    return cudaGetLastError();
}

cudaError_t infer_silu_mul_halves_clamped_f32_batch_on_stream(const float* gate_up, float* output, uint32_t rows, uint32_t cols,
                                                              float limit, cudaStream_t stream) {
    if (!gate_up || !output || rows == 0 || cols == 0 || !isfinite(limit) || limit <= 0.0f) return cudaErrorInvalidValue;
    const size_t len = static_cast<size_t>(rows) * cols;
    act_mul_f32_kernel<kSiluHalves><<<static_cast<uint32_t>((len + 255) / 256), 256, 0, stream>>>(gate_up, nullptr, output, rows, cols, limit);
    return cudaGetLastError();
}

cudaError_t infer_silu_mul_halves_clamped_f32_on_stream(const float* gate_up, float* output, uint32_t len, float limit,
                                                        cudaStream_t stream) {
    return infer_silu_mul_halves_clamped_f32_batch_on_stream(gate_up, output, 1, len, limit, stream);
}

cudaError_t infer_silu_mul_halves_f32_on_stream(const float* gate_up, float* output, uint32_t len, cudaStream_t stream) {
    return infer_silu_mul_halves_f32_batch_on_stream(gate_up, output, 1, len, stream);
}

cudaError_t infer_gelu_tanh_mul_f32_on_stream(const float* gate, const float* up, float* output, uint32_t len,
                                              cudaStream_t stream) {
    if (!gate || !up || !output || len == 0) return cudaErrorInvalidValue;
    act_mul_f32_kernel<kGeluPair><<<(len + 255) / 256, 256, 0, stream>>>(gate, up, output, 1, len, 0.0f);
    return cudaGetLastError();
}

cudaError_t infer_unpack_heads_f32_on_stream(const float* input, float* output, uint32_t tokens, uint32_t heads,
                                             uint32_t head_dim, uint32_t output_row_offset, cudaStream_t stream) {
    if (!input || !output || tokens == 0 || heads == 0 || head_dim == 0) return cudaErrorInvalidValue;
    const size_t total = static_cast<size_t>(tokens) * heads * head_dim;
    unpack_heads_f32_kernel<<<static_cast<uint32_t>((total + 255) / 256), 256, 0, stream>>>(input, output, tokens, heads, head_dim,
                                                                                           output_row_offset);
    return cudaGetLastError();
}

cudaError_t infer_scale_channel_f32_device_scalar_on_stream(float* values, const float* channel_scale, const float* scalar,
                                                            uint32_t len, cudaStream_t stream) {
    if (!values || !channel_scale || !scalar || len == 0) return cudaErrorInvalidValue;
    scale_channel_kernel<<<(len + 255) / 256, 256, 0, stream>>>(values, channel_scale, scalar, len, len, 0);
    return cudaGetLastError();
}

cudaError_t infer_scale_channel_f32_device_row_scalar_on_stream(float* values, const float* channel_scale,
                                                                const float* row_scale, uint32_t rows, uint32_t channels,
                                                                cudaStream_t stream) {
    if (!values || !channel_scale || !row_scale || rows == 0 || channels == 0) return cudaErrorInvalidValue;
    const size_t len = static_cast<size_t>(rows) * channels;
    scale_channel_kernel<<<static_cast<uint32_t>((len + 255) / 256), 256, 0, stream>>>(values, channel_scale, row_scale, channels,
                                                                                      len, 1);
    return cudaGetLastError();
}

cudaError_t infer_gelu_tanh_mul_quantize_nvfp4_col_major_f32_on_stream(const float* gate, const float* up, uint8_t* packed,
                                                                       uint8_t* scales, uint32_t rows, uint32_t cols,
                                                                       float input_scale, cudaStream_t stream) {
    if (!gate || !up || !packed || !scales || rows == 0 || cols == 0 || cols % 16 != 0 || bad_scale(input_scale) ||
        !aligned16(gate, up) || (reinterpret_cast<uintptr_t>(packed) & 7) != 0)
        return cudaErrorInvalidValue;
    const dim3 grid((cols / 16 + 255) / 256, rows);
    gelu_mul_quantize_kernel<<<grid, 256, 0, stream>>>(gate, up, packed, scales, cols, input_scale);
    return cudaGetLastError();
}

static cudaError_t unpack_heads_quantize(const void* input, int is_bf16, uint8_t* packed, uint8_t* scales, uint32_t tokens,
                                         uint32_t heads, uint32_t head_dim, uint32_t output_row_offset, float input_scale,
                                         cudaStream_t stream) {
    if (!input || !packed || !scales || tokens == 0 || heads == 0 || head_dim == 0 || head_dim % 16 != 0 ||
        bad_scale(input_scale) || (reinterpret_cast<uintptr_t>(packed) & 7) != 0)
        return cudaErrorInvalidValue;
    const dim3 grid((heads * head_dim / 16 + 127) / 128, tokens);
    if (is_bf16)
        unpack_heads_quantize_kernel<uint16_t><<<grid, 128, 0, stream>>>(static_cast<const uint16_t*>(input), packed, scales, tokens,
                                                                       heads, head_dim, output_row_offset, input_scale);
    else
        unpack_heads_quantize_kernel<float><<<grid, 128, 0, stream>>>(static_cast<const float*>(input), packed, scales, tokens, heads,
                                                                    head_dim, output_row_offset, input_scale);
    return cudaGetLastError();
}

cudaError_t infer_unpack_heads_quantize_nvfp4_col_major_f32_on_stream(const float* input, uint8_t* packed, uint8_t* scales,
                                                                      uint32_t tokens, uint32_t heads, uint32_t head_dim,
                                                                      uint32_t output_row_offset, float input_scale,
                                                                      cudaStream_t stream) {
    return unpack_heads_quantize(input, 0, packed, scales, tokens, heads, head_dim, output_row_offset, input_scale, stream);
}

cudaError_t infer_unpack_heads_quantize_nvfp4_col_major_bf16_on_stream(const uint16_t* input, uint8_t* packed, uint8_t* scales,
                                                                       uint32_t tokens, uint32_t heads, uint32_t head_dim,
                                                                       uint32_t output_row_offset, float input_scale,
                                                                       cudaStream_t stream) {
    return unpack_heads_quantize(input, 1, packed, scales, tokens, heads, head_dim, output_row_offset, input_scale, stream);
}

cudaError_t infer_gated_rms_norm_quantize_nvfp4_col_major_f32_on_stream(const float* input, const float* gate, const float* weight,
                                                                        uint8_t* packed, uint8_t* scales, uint32_t rows,
                                                                        uint32_t heads, uint32_t head_dim, float eps,
                                                                        float input_scale, cudaStream_t stream) {
    if (!input || !gate || !weight || !packed || !scales || rows == 0 || heads == 0 || head_dim != 128 || bad_scale(input_scale) ||
        (reinterpret_cast<uintptr_t>(packed) & 7) != 0)
        return cudaErrorInvalidValue;
    gated_rms_norm_quantize_kernel<<<rows * heads, 128, 0, stream>>>(input, gate, weight, packed, scales, heads, eps, input_scale);
    return cudaGetLastError();
}

cudaError_t infer_quantize_nvfp4_vector_simple_scales_f32_on_stream(const float* input, uint8_t* packed, uint8_t* scales,
                                                                    uint32_t rows, float input_scale, cudaStream_t stream) {
    if (!input || !packed || !scales || rows == 0 || bad_scale(input_scale)) return cudaErrorInvalidValue;
    const uint32_t blocks = (rows + 15) / 16;
    quantize_vector_simple_scales_kernel<<<(blocks + 127) / 128, 128, 0, stream>>>(input, packed, scales, rows, input_scale);
    return cudaGetLastError();
}

}  // extern "C"
