// CUDA-core decode kernels that keep the reference's exact f32 semantics:
//   * W4A16 GEMV  y[b][n] = w2 * sum_k x[b][k] * e2m1(W[n][k]) * e4m3(S[n][k/16])
//     (crates/eider-cuda/native/non_gemm.cu:13147-13256), row-major checkpoint scales read directly;
//   * FP8 W8A8 linear for a few tokens, y[b][n] = (sum_k e4m3(xq) * e4m3(w)) * s_x[b] * s_w[n]
//     (crates/eider-cuda/native/non_gemm.cu:9976-10011).
// Both stream the weight matrix once with 128-bit loads, one warp per output row, activations staged
// in shared memory, warp-shuffle reduction.  HBM-bound; the tensor-core decode path lives in
// gemm_umma.cu and these kernels serve shapes it does not take and f32-in/f32-out callers.
#include "common.cuh"
#include "eider_b200.h"

namespace eider {
namespace {

constexpr int kWarpsPerBlock = 8;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Shared-memory position of element `e` (0..31) of 32-element chunk `c`: float4 slots are XOR-swizzled
// by the chunk index so that lanes reading the same slot of consecutive chunks hit distinct banks.
__device__ __forceinline__ uint32_t xs_index(uint32_t c, uint32_t e) {
    return c * 32 + ((((e >> 2) ^ (c & 7u)) << 2) | (e & 3u));
}

template <typename XT> __device__ __forceinline__ float load_x(const XT* p);
template <> __device__ __forceinline__ float load_x<float>(const float* p) { return __ldg(p); }
template <> __device__ __forceinline__ float load_x<uint16_t>(const uint16_t* p) { return bf16_bits_to_float(__ldg(p)); }

template <typename YT> __device__ __forceinline__ void store_y(YT* p, float v);
template <> __device__ __forceinline__ void store_y<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void store_y<uint16_t>(uint16_t* p, float v) { *p = float_to_bf16_bits(v); }

__device__ __forceinline__ void dot_word(uint32_t w, const float* xs, uint32_t c, uint32_t e0, float& acc) {
    float4 a = *reinterpret_cast<const float4*>(xs + xs_index(c, e0));
    float4 b = *reinterpret_cast<const float4*>(xs + xs_index(c, e0 + 4));
    acc = fmaf(e2m1_value(w), a.x, acc);
    acc = fmaf(e2m1_value(w >> 4), a.y, acc);
    acc = fmaf(e2m1_value(w >> 8), a.z, acc);
    acc = fmaf(e2m1_value(w >> 12), a.w, acc);
    acc = fmaf(e2m1_value(w >> 16), b.x, acc);
    acc = fmaf(e2m1_value(w >> 20), b.y, acc);
    acc = fmaf(e2m1_value(w >> 24), b.z, acc);
    acc = fmaf(e2m1_value(w >> 28), b.w, acc);
}

template <int B, typename XT, typename YT>
__global__ void __launch_bounds__(kWarpsPerBlock * 32) w4a16_gemv_kernel(const XT* __restrict__ x,
                                                                         const uint8_t* __restrict__ w,
                                                                         const uint8_t* __restrict__ s,
                                                                         YT* __restrict__ y, uint32_t n, uint32_t k,
                                                                         float w2) {
    extern __shared__ float xs[];  // [B][chunks * 32], swizzled
    const uint32_t chunks = (k + 31) / 32;
    const uint32_t kpad = chunks * 32;
    for (uint32_t i = threadIdx.x; i < B * kpad; i += blockDim.x) {
        uint32_t b = i / kpad, e = i % kpad;
        xs[b * kpad + xs_index(e / 32, e % 32)] = e < k ? load_x<XT>(x + static_cast<size_t>(b) * k + e) : 0.0f;
    }
    __syncthreads();
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t row = blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
    if (row >= n) return;
    const uint8_t* wrow = w + static_cast<size_t>(row) * (k / 2);
    const uint8_t* srow = s + static_cast<size_t>(row) * (k / 16);
    const bool aligned32 = (k % 32 == 0);
    float acc[B];
#pragma unroll
    for (int b = 0; b < B; ++b) acc[b] = 0.0f;
    for (uint32_t c = lane; c < chunks; c += 32) {
        const bool full = (c * 32 + 32) <= k;
        uint4 q;
        float s0, s1;
        if (aligned32) {  // rows start on 16-byte boundaries: one 128-bit load + one 16-bit scale pair
            q = __ldg(reinterpret_cast<const uint4*>(wrow + c * 16));
            uint16_t sc = __ldg(reinterpret_cast<const uint16_t*>(srow + c * 2));
            s0 = e4m3_value(static_cast<uint8_t>(sc & 0xff));
            s1 = e4m3_value(static_cast<uint8_t>(sc >> 8));
        } else {  // k % 32 == 16: rows are only 8-byte aligned and the last chunk has one block
            uint2 h0 = __ldg(reinterpret_cast<const uint2*>(wrow + c * 16));
            uint2 h1 = full ? __ldg(reinterpret_cast<const uint2*>(wrow + c * 16 + 8)) : make_uint2(0u, 0u);
            q = make_uint4(h0.x, h0.y, h1.x, h1.y);
            s0 = e4m3_value(__ldg(srow + c * 2));
            s1 = full ? e4m3_value(__ldg(srow + c * 2 + 1)) : 0.0f;
        }
#pragma unroll
        for (int b = 0; b < B; ++b) {
            const float* xb = xs + b * kpad;
            float p0 = 0.0f, p1 = 0.0f;
            dot_word(q.x, xb, c, 0, p0);
            dot_word(q.y, xb, c, 8, p0);
            dot_word(q.z, xb, c, 16, p1);
            dot_word(q.w, xb, c, 24, p1);
            acc[b] = fmaf(s0, p0, acc[b]);
            acc[b] = fmaf(s1, p1, acc[b]);
        }
    }
#pragma unroll
    for (int b = 0; b < B; ++b) {
        float v = warp_sum(acc[b]);
        if (lane == 0) store_y<YT>(y + static_cast<size_t>(b) * n + row, v * w2);
    }
}

template <typename XT, typename YT>
cudaError_t launch_w4a16(const XT* x, const uint8_t* w, const uint8_t* s, YT* y, uint32_t batch, uint32_t n,
                         uint32_t k, float w2, cudaStream_t stream) {
    if (!x || !w || !s || !y || batch == 0 || n == 0 || k == 0 || k % 16 != 0) return cudaErrorInvalidValue;
    const uint32_t kpad = (k + 31) / 32 * 32;
    const uint32_t grid = (n + kWarpsPerBlock - 1) / kWarpsPerBlock;
    uint32_t done = 0;
    while (done < batch) {
        uint32_t b = batch - done >= 4 ? 4 : (batch - done >= 2 ? 2 : 1);
        size_t smem = static_cast<size_t>(b) * kpad * sizeof(float);
        if (smem > 200 * 1024) return cudaErrorNotSupported;
        const XT* xb = x + static_cast<size_t>(done) * k;
        YT* yb = y + static_cast<size_t>(done) * n;
        cudaError_t st = cudaSuccess;
#define EIDER_LAUNCH_W4A16(BB)                                                                                   \
    do {                                                                                                         \
        if (smem > 48 * 1024)                                                                                    \
            st = cudaFuncSetAttribute(w4a16_gemv_kernel<BB, XT, YT>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                      static_cast<int>(smem));                                                   \
        if (st == cudaSuccess)                                                                                   \
            w4a16_gemv_kernel<BB, XT, YT><<<grid, kWarpsPerBlock * 32, smem, stream>>>(xb, w, s, yb, n, k, w2);  \
    } while (0)
        if (b == 4) EIDER_LAUNCH_W4A16(4);
        else if (b == 2) EIDER_LAUNCH_W4A16(2);
        else EIDER_LAUNCH_W4A16(1);
#undef EIDER_LAUNCH_W4A16
        if (st != cudaSuccess) return st;
        st = cudaGetLastError();
        if (st != cudaSuccess) return st;
        done += b;
    }
    return cudaSuccess;
}

// FP8 weights [N][K] bytes, activations already quantized per token.
template <int B, typename YT>
__global__ void __launch_bounds__(kWarpsPerBlock * 32) fp8_linear_simt_kernel(const uint8_t* __restrict__ xq,
                                                                              const float* __restrict__ s_x,
                                                                              const uint8_t* __restrict__ w,
                                                                              const float* __restrict__ s_w,
                                                                              float s_w_scalar, YT* __restrict__ y,
                                                                              uint32_t n, uint32_t k) {
    extern __shared__ float xs[];  // [B][k] decoded activations, 16-element chunks swizzled like above
    const uint32_t chunks = (k + 31) / 32;
    const uint32_t kpad = chunks * 32;
    for (uint32_t i = threadIdx.x; i < B * kpad; i += blockDim.x) {
        uint32_t b = i / kpad, e = i % kpad;
        xs[b * kpad + xs_index(e / 32, e % 32)] = e < k ? e4m3_value(__ldg(xq + static_cast<size_t>(b) * k + e)) : 0.0f;
    }
    __syncthreads();
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t row = blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
    if (row >= n) return;
    const uint8_t* wrow = w + static_cast<size_t>(row) * k;
    float acc[B];
#pragma unroll
    for (int b = 0; b < B; ++b) acc[b] = 0.0f;
    const bool vec_ok = (k % 16 == 0);
    // 16 weights per lane per step; two steps cover one 32-element chunk
    for (uint32_t h = lane; h < (k + 15) / 16; h += 32) {
        uint32_t c = h / 2, e0 = (h & 1) * 16;
        float wv[16];
        if (vec_ok) {
            uint4 q = __ldg(reinterpret_cast<const uint4*>(wrow + h * 16));
            uint32_t ww[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
            for (int j = 0; j < 4; ++j)
#pragma unroll
                for (int i = 0; i < 4; ++i) wv[4 * j + i] = e4m3_value(static_cast<uint8_t>(ww[j] >> (8 * i)));
        } else {
#pragma unroll
            for (int i = 0; i < 16; ++i) wv[i] = (h * 16 + i) < k ? e4m3_value(__ldg(wrow + h * 16 + i)) : 0.0f;
        }
#pragma unroll
        for (int b = 0; b < B; ++b) {
            const float* xb = xs + b * kpad;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                float4 a = *reinterpret_cast<const float4*>(xb + xs_index(c, e0 + 4 * j));
                acc[b] = fmaf(wv[4 * j], a.x, acc[b]);
                acc[b] = fmaf(wv[4 * j + 1], a.y, acc[b]);
                acc[b] = fmaf(wv[4 * j + 2], a.z, acc[b]);
                acc[b] = fmaf(wv[4 * j + 3], a.w, acc[b]);
            }
        }
    }
    const float sw = s_w ? __ldg(s_w + row) : s_w_scalar;
#pragma unroll
    for (int b = 0; b < B; ++b) {
        float v = warp_sum(acc[b]);
        if (lane == 0) store_y<YT>(y + static_cast<size_t>(b) * n + row, v * __ldg(s_x + b) * sw);
    }
}

template <typename YT>
cudaError_t launch_fp8_simt(const uint8_t* xq, const float* s_x, const uint8_t* w, const float* s_w, float s_w_scalar,
                            YT* y, uint32_t m, uint32_t n, uint32_t k, cudaStream_t stream) {
    if (!xq || !s_x || !w || !y || m == 0 || n == 0 || k == 0) return cudaErrorInvalidValue;
    const uint32_t kpad = (k + 31) / 32 * 32;
    const uint32_t grid = (n + kWarpsPerBlock - 1) / kWarpsPerBlock;
    uint32_t done = 0;
    while (done < m) {
        uint32_t b = m - done >= 4 ? 4 : (m - done >= 2 ? 2 : 1);
        size_t smem = static_cast<size_t>(b) * kpad * sizeof(float);
        if (smem > 200 * 1024) return cudaErrorNotSupported;
        const uint8_t* xb = xq + static_cast<size_t>(done) * k;
        YT* yb = y + static_cast<size_t>(done) * n;
        cudaError_t st = cudaSuccess;
#define EIDER_LAUNCH_FP8(BB)                                                                                       \
    do {                                                                                                           \
        if (smem > 48 * 1024)                                                                                      \
            st = cudaFuncSetAttribute(fp8_linear_simt_kernel<BB, YT>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                      static_cast<int>(smem));                                                     \
        if (st == cudaSuccess)                                                                                     \
            fp8_linear_simt_kernel<BB, YT><<<grid, kWarpsPerBlock * 32, smem, stream>>>(xb, s_x + done, w, s_w,    \
                                                                                        s_w_scalar, yb, n, k);     \
    } while (0)
        if (b == 4) EIDER_LAUNCH_FP8(4);
        else if (b == 2) EIDER_LAUNCH_FP8(2);
        else EIDER_LAUNCH_FP8(1);
#undef EIDER_LAUNCH_FP8
        if (st != cudaSuccess) return st;
        st = cudaGetLastError();
        if (st != cudaSuccess) return st;
        done += b;
    }
    return cudaSuccess;
}

// Block-scaled FP8 linear for a few tokens (crates/eider-cuda/native/deepseek4.cu:86-115, 117-170): weights [N][K] E4M3 with
// one scale per 128 x 128 block, either an E8M0 byte or an f32; y[b][n] = sum_k x[b][k] * e4m3(w[n][k]) * scale[n/128][k/128]
// with f32 activations (no activation quantization).  Same streaming shape as the kernels above: one warp per output row,
// 128-bit weight loads (16 weights, always inside one scale block), activations of up to four tokens staged in shared
// memory, so the weight matrix is read once per four tokens.
template <int B, typename ScaleT>
__global__ void __launch_bounds__(kWarpsPerBlock * 32) block_fp8_linear_kernel(const float* __restrict__ x, const uint8_t* __restrict__ w,
                                                                               const ScaleT* __restrict__ scales, float* __restrict__ y,
                                                                               uint32_t n, uint32_t k) {
    extern __shared__ float xs[];  // [B][k], 32-element chunks swizzled
    for (uint32_t i = threadIdx.x; i < B * k; i += blockDim.x) {
        const uint32_t b = i / k, e = i % k;
        xs[b * k + xs_index(e / 32, e % 32)] = __ldg(x + static_cast<size_t>(b) * k + e);
    }
    __syncthreads();
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t row = blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
    if (row >= n) return;
    const uint8_t* wrow = w + static_cast<size_t>(row) * k;
    const ScaleT* srow = scales + static_cast<size_t>(row / 128) * (k / 128);
    float acc[B];
#pragma unroll
    for (int b = 0; b < B; ++b) acc[b] = 0.0f;
    for (uint32_t h = lane; h < k / 16; h += 32) {
        const uint4 q = __ldg(reinterpret_cast<const uint4*>(wrow + h * 16));
        const uint32_t ww[4] = {q.x, q.y, q.z, q.w};
        float scale;
        if constexpr (sizeof(ScaleT) == 1) {
            const uint32_t code = __ldg(reinterpret_cast<const uint8_t*>(srow) + h / 8);
            scale = code == 255 ? __int_as_float(0x7fc00000) : (code == 0 ? __int_as_float(0x00400000) : __int_as_float(code << 23));  // 2^(code - 127)
        } else {
            scale = __ldg(reinterpret_cast<const float*>(srow) + h / 8);
        }
        const uint32_t c = h / 2, e0 = (h & 1) * 16;
#pragma unroll
        for (int b = 0; b < B; ++b) {
            const float* xb = xs + b * k;
            float part = 0.0f;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float4 a = *reinterpret_cast<const float4*>(xb + xs_index(c, e0 + 4 * j));
                part = fmaf(e4m3_value(static_cast<uint8_t>(ww[j])), a.x, part);
                part = fmaf(e4m3_value(static_cast<uint8_t>(ww[j] >> 8)), a.y, part);
                part = fmaf(e4m3_value(static_cast<uint8_t>(ww[j] >> 16)), a.z, part);
                part = fmaf(e4m3_value(static_cast<uint8_t>(ww[j] >> 24)), a.w, part);
            }
            acc[b] = fmaf(scale, part, acc[b]);
        }
    }
#pragma unroll
    for (int b = 0; b < B; ++b) {
        const float v = warp_sum(acc[b]);
        if (lane == 0) y[static_cast<size_t>(b) * n + row] = v;
    }
}

template <typename ScaleT>
cudaError_t launch_block_fp8(const float* x, const uint8_t* w, const ScaleT* scales, float* y, uint32_t batch, uint32_t n, uint32_t k,
                             cudaStream_t stream) {
    if (!x || !w || !scales || !y || batch == 0 || n == 0 || k == 0 || n % 128 != 0 || k % 128 != 0) return cudaErrorInvalidValue;
    const uint32_t grid = (n + kWarpsPerBlock - 1) / kWarpsPerBlock;
    uint32_t done = 0;
    while (done < batch) {
        const uint32_t b = batch - done >= 4 ? 4 : (batch - done >= 2 ? 2 : 1);
        const size_t smem = static_cast<size_t>(b) * k * sizeof(float);
        if (smem > 200 * 1024) return cudaErrorNotSupported;
        const float* xb = x + static_cast<size_t>(done) * k;
        float* yb = y + static_cast<size_t>(done) * n;
        cudaError_t st = cudaSuccess;
#define EIDER_LAUNCH_BLOCK_FP8(BB)                                                                                             \
    do {                                                                                                                       \
        if (smem > 48 * 1024)                                                                                                  \
            st = cudaFuncSetAttribute(block_fp8_linear_kernel<BB, ScaleT>, cudaFuncAttributeMaxDynamicSharedMemorySize,       \
                                      static_cast<int>(smem));                                                                 \
        if (st == cudaSuccess) block_fp8_linear_kernel<BB, ScaleT><<<grid, kWarpsPerBlock * 32, smem, stream>>>(xb, w, scales, yb, n, k); \
    } while (0)
        if (b == 4) EIDER_LAUNCH_BLOCK_FP8(4);
        else if (b == 2) EIDER_LAUNCH_BLOCK_FP8(2);
        else EIDER_LAUNCH_BLOCK_FP8(1);
#undef EIDER_LAUNCH_BLOCK_FP8
        if (st != cudaSuccess) return st;
        st = cudaGetLastError();
        if (st != cudaSuccess) return st;
        done += b;
    }
    return cudaSuccess;
}

// FP8 weight-only linear for a few tokens (crates/eider-cuda/native/non_gemm.cu:9642-9684): y[b][n] = scale(n) * sum_k x[b][k] *
// e4m3(w[n][k]) with f32 activations and either one weight scale or one per output row.  QUANT_X is the "precomputed
// dynamic" form (non_gemm.cu:9900-9925): the activation is replaced by e4m3(x / s_x) with the per-tensor s_x a preceding
// kernel has written, and the result is multiplied by s_x.  Same streaming shape as the kernels above.
template <int B, bool QUANT_X>
__global__ void __launch_bounds__(kWarpsPerBlock * 32) fp8_weight_only_kernel(const float* __restrict__ x, const uint8_t* __restrict__ w,
                                                                              const float* __restrict__ channel_scale, float weight_scale,
                                                                              const float* __restrict__ x_scale, float* __restrict__ y,
                                                                              uint32_t n, uint32_t k) {
    extern __shared__ float xs[];  // [B][kpad], 32-element chunks swizzled
    const uint32_t kpad = (k + 31) / 32 * 32;
    const float sx = QUANT_X ? __ldg(x_scale) : 1.0f;
    for (uint32_t i = threadIdx.x; i < B * k; i += blockDim.x) {
        const uint32_t b = i / k, e = i % k;
        float v = __ldg(x + static_cast<size_t>(b) * k + e);
        if (QUANT_X) v = e4m3_value(e4m3_satfinite(__fdiv_rn(v, sx)));
        xs[b * kpad + xs_index(e / 32, e % 32)] = v;
    }
    __syncthreads();
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t row = blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
    if (row >= n) return;
    const uint8_t* wrow = w + static_cast<size_t>(row) * k;
    float acc[B];
#pragma unroll
    for (int b = 0; b < B; ++b) acc[b] = 0.0f;
    for (uint32_t h = lane; h < k / 16; h += 32) {
        const uint4 q = __ldg(reinterpret_cast<const uint4*>(wrow + h * 16));
        const uint32_t ww[4] = {q.x, q.y, q.z, q.w};
        float wv[16];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            wv[4 * j] = e4m3_value(static_cast<uint8_t>(ww[j]));
            wv[4 * j + 1] = e4m3_value(static_cast<uint8_t>(ww[j] >> 8));
            wv[4 * j + 2] = e4m3_value(static_cast<uint8_t>(ww[j] >> 16));
            wv[4 * j + 3] = e4m3_value(static_cast<uint8_t>(ww[j] >> 24));
        }
        const uint32_t c = h / 2, e0 = (h & 1) * 16;
#pragma unroll
        for (int b = 0; b < B; ++b) {
            const float* xb = xs + b * kpad;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float4 a = *reinterpret_cast<const float4*>(xb + xs_index(c, e0 + 4 * j));
                acc[b] = fmaf(wv[4 * j], a.x, acc[b]);
                acc[b] = fmaf(wv[4 * j + 1], a.y, acc[b]);
                acc[b] = fmaf(wv[4 * j + 2], a.z, acc[b]);
                acc[b] = fmaf(wv[4 * j + 3], a.w, acc[b]);
            }
        }
    }
    const float scale = (channel_scale ? __ldg(channel_scale + row) : weight_scale) * sx;
#pragma unroll
    for (int b = 0; b < B; ++b) {
        const float v = warp_sum(acc[b]);
        if (lane == 0) y[static_cast<size_t>(b) * n + row] = v * scale;
    }
}

// amax / 448 of one activation row (1 when it is all zero), as the per-token quantizer computes it (non_gemm.cu:9880-9898)
__global__ void __launch_bounds__(256) fp8_input_scale_kernel(const float* __restrict__ x, float* __restrict__ scale, uint32_t k) {
    __shared__ float red[8];
    float amax = 0.0f;
    for (uint32_t i = threadIdx.x; i < k; i += 256) amax = fmaxf(amax, fabsf(__ldg(x + i)));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 16));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 8));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int i = 1; i < 8; ++i) amax = fmaxf(amax, red[i]);
        scale[0] = amax == 0.0f ? 1.0f : __fdiv_rn(amax, 448.0f);
    }
}

template <bool QUANT_X>
cudaError_t launch_fp8_weight_only(const float* x, const uint8_t* w, const float* channel_scale, float weight_scale, const float* x_scale,
                                   float* y, uint32_t batch, uint32_t n, uint32_t k, cudaStream_t stream) {
    if (!x || !w || !y || batch == 0 || n == 0 || k == 0 || k % 16 != 0 || !isfinite(weight_scale) ||
        ((reinterpret_cast<uintptr_t>(w)) & 15) != 0)
        return cudaErrorInvalidValue;
    const uint32_t grid = (n + kWarpsPerBlock - 1) / kWarpsPerBlock;
    uint32_t done = 0;
    while (done < batch) {
        const uint32_t b = batch - done >= 4 ? 4 : (batch - done >= 2 ? 2 : 1);
        const size_t smem = static_cast<size_t>(b) * ((k + 31) / 32 * 32) * sizeof(float);
        if (smem > 200 * 1024) return cudaErrorNotSupported;
        const float* xb = x + static_cast<size_t>(done) * k;
        float* yb = y + static_cast<size_t>(done) * n;
        cudaError_t st = cudaSuccess;
#define EIDER_LAUNCH_FP8_WO(BB)                                                                                                \
    do {                                                                                                                       \
        if (smem > 48 * 1024)                                                                                                  \
            st = cudaFuncSetAttribute(fp8_weight_only_kernel<BB, QUANT_X>, cudaFuncAttributeMaxDynamicSharedMemorySize,        \
                                      static_cast<int>(smem));                                                                 \
        if (st == cudaSuccess)                                                                                                 \
            fp8_weight_only_kernel<BB, QUANT_X><<<grid, kWarpsPerBlock * 32, smem, stream>>>(xb, w, channel_scale, weight_scale, \
                                                                                             x_scale, yb, n, k);               \
    } while (0)
        if (b == 4) EIDER_LAUNCH_FP8_WO(4);
        else if (b == 2) EIDER_LAUNCH_FP8_WO(2);
        else EIDER_LAUNCH_FP8_WO(1);
#undef EIDER_LAUNCH_FP8_WO
        if (st != cudaSuccess) return st;
        st = cudaGetLastError();
        if (st != cudaSuccess) return st;
        done += b;
    }
    return cudaSuccess;
}

bool bad_threads(uint32_t threads) { return threads < 64 || threads > 512 || threads % 32 != 0; }  // (validated as the reference does; not used)

}  // namespace
}  // namespace eider

using namespace eider;

extern "C" {

// ---- FP8 weight-only linears of the reference (crates/eider-cuda/src/ffi.rs:3056-3147; kernels non_gemm.cu:9642-9950) ------
cudaError_t infer_fp8_linear_f32_batch_on_stream(const float* input, const uint8_t* weight, float* output, uint32_t batch_size,
                                                 uint32_t rows, uint32_t cols, float weight_scale, uint32_t threads, cudaStream_t stream) {
    if (bad_threads(threads)) return cudaErrorInvalidValue;
    return launch_fp8_weight_only<false>(input, weight, nullptr, weight_scale, nullptr, output, batch_size, rows, cols, stream);
}

cudaError_t infer_fp8_linear_f32_configured_on_stream(const float* input, const uint8_t* weight, float* output, uint32_t rows,
                                                      uint32_t cols, float weight_scale, uint32_t threads, cudaStream_t stream) {
    return infer_fp8_linear_f32_batch_on_stream(input, weight, output, 1, rows, cols, weight_scale, threads, stream);
}

cudaError_t infer_fp8_linear_pair_f32_configured_on_stream(const float* input, const uint8_t* first_weight, const uint8_t* second_weight,
                                                           float* first_output, float* second_output, uint32_t first_rows,
                                                           uint32_t second_rows, uint32_t cols, float first_scale, float second_scale,
                                                           uint32_t threads, cudaStream_t stream) {
    if (!input || !first_weight || !second_weight || !first_output || !second_output || first_rows == 0 || second_rows == 0 ||
        cols == 0 || !isfinite(first_scale) || !isfinite(second_scale) || bad_threads(threads))
        return cudaErrorInvalidValue;
    cudaError_t st = launch_fp8_weight_only<false>(input, first_weight, nullptr, first_scale, nullptr, first_output, 1, first_rows, cols, stream);
    if (st != cudaSuccess) return st;
    return launch_fp8_weight_only<false>(input, second_weight, nullptr, second_scale, nullptr, second_output, 1, second_rows, cols, stream);
}

cudaError_t infer_fp8_linear_triple_f32_configured_on_stream(const float* input, const uint8_t* first_weight, const uint8_t* second_weight,
                                                             const uint8_t* third_weight, float* first_output, float* second_output,
                                                             float* third_output, uint32_t first_rows, uint32_t second_rows,
                                                             uint32_t third_rows, uint32_t cols, float first_scale, float second_scale,
                                                             float third_scale, uint32_t threads, cudaStream_t stream) {
    if (!third_weight || !third_output || third_rows == 0 || !isfinite(third_scale)) return cudaErrorInvalidValue;
    cudaError_t st = infer_fp8_linear_pair_f32_configured_on_stream(input, first_weight, second_weight, first_output, second_output,
                                                                    first_rows, second_rows, cols, first_scale, second_scale, threads, stream);
    if (st != cudaSuccess) return st;
    return launch_fp8_weight_only<false>(input, third_weight, nullptr, third_scale, nullptr, third_output, 1, third_rows, cols, stream);
}

cudaError_t infer_fp8_linear_channel_scaled_f32_batch_configured_on_stream(const float* input, const uint8_t* weight,
                                                                           const float* channel_weight_scale, float* output,
                                                                           uint32_t batch_size, uint32_t rows, uint32_t cols,
                                                                           uint32_t threads, cudaStream_t stream) {
    if (!channel_weight_scale || bad_threads(threads)) return cudaErrorInvalidValue;
    return launch_fp8_weight_only<false>(input, weight, channel_weight_scale, 1.0f, nullptr, output, batch_size, rows, cols, stream);
}

cudaError_t infer_fp8_linear_channel_scaled_f32_configured_on_stream(const float* input, const uint8_t* weight,
                                                                     const float* channel_weight_scale, float* output, uint32_t rows,
                                                                     uint32_t cols, uint32_t threads, cudaStream_t stream) {
    return infer_fp8_linear_channel_scaled_f32_batch_configured_on_stream(input, weight, channel_weight_scale, output, 1, rows, cols, threads,
                                                                          stream);
}

cudaError_t infer_fp8_linear_channel_scaled_precomputed_dynamic_f32_on_stream(const float* input, const uint8_t* weight,
                                                                              const float* channel_weight_scale, float* input_scale,
                                                                              float* output, uint32_t rows, uint32_t cols,
                                                                              cudaStream_t stream) {
    if (!input || !weight || !channel_weight_scale || !input_scale || !output || rows == 0 || cols == 0) return cudaErrorInvalidValue;
    fp8_input_scale_kernel<<<1, 256, 0, stream>>>(input, input_scale, cols);
    cudaError_t st = cudaGetLastError();
    if (st != cudaSuccess) return st;
    return launch_fp8_weight_only<true>(input, weight, channel_weight_scale, 1.0f, input_scale, output, 1, rows, cols, stream);
}


cudaError_t infer_nvfp4_w4a16_matvec_f32_on_stream(const float* input, const uint8_t* packed_weight,
                                                   const uint8_t* weight_scale, float* output, uint32_t out_features,
                                                   uint32_t in_features, float weight_scale_2, cudaStream_t stream) {
    return launch_w4a16<float, float>(input, packed_weight, weight_scale, output, 1, out_features, in_features,
                                      weight_scale_2, stream);
}

cudaError_t infer_nvfp4_w4a16_matvec_f32_warp_rows_on_stream(const float* input, const uint8_t* packed_weight,
                                                             const uint8_t* weight_scale, float* output, uint32_t out_features,
                                                             uint32_t in_features, float weight_scale_2, uint32_t warps_per_block,
                                                             cudaStream_t stream) {
    (void)warps_per_block;  // launch geometry is fixed here; kept for signature compatibility
    return launch_w4a16<float, float>(input, packed_weight, weight_scale, output, 1, out_features, in_features, weight_scale_2, stream);
}

cudaError_t infer_nvfp4_w4a16_matvec_f32_warp_rows_batch_on_stream(const float* input, const uint8_t* packed_weight,
                                                                   const uint8_t* weight_scale, float* output,
                                                                   uint32_t batch_size, uint32_t out_features,
                                                                   uint32_t in_features, float weight_scale_2,
                                                                   uint32_t warps_per_block, cudaStream_t stream) {
    (void)warps_per_block;  // launch geometry is fixed here; kept for signature compatibility
    return launch_w4a16<float, float>(input, packed_weight, weight_scale, output, batch_size, out_features,
                                      in_features, weight_scale_2, stream);
}

cudaError_t eider_b200_nvfp4_w4a16_matvec_bf16_on_stream(const uint16_t* input, const uint8_t* packed_weight,
                                                         const uint8_t* weight_scale, uint16_t* output,
                                                         uint32_t batch_size, uint32_t out_features,
                                                         uint32_t in_features, float weight_scale_2,
                                                         cudaStream_t stream) {
    return launch_w4a16<uint16_t, uint16_t>(input, packed_weight, weight_scale, output, batch_size, out_features,
                                            in_features, weight_scale_2, stream);
}

cudaError_t eider_b200_fp8_linear_prequantized_simt_on_stream(const uint8_t* xq, const float* input_scales,
                                                              const uint8_t* weight, const float* channel_scale,
                                                              float weight_scale, void* output, int output_is_bf16,
                                                              uint32_t tokens, uint32_t out_features,
                                                              uint32_t in_features, cudaStream_t stream) {
    if (output_is_bf16)
        return launch_fp8_simt<uint16_t>(xq, input_scales, weight, channel_scale, weight_scale,
                                         static_cast<uint16_t*>(output), tokens, out_features, in_features, stream);
    return launch_fp8_simt<float>(xq, input_scales, weight, channel_scale, weight_scale, static_cast<float*>(output),
                                  tokens, out_features, in_features, stream);
}

cudaError_t infer_deepseek4_block_fp8_linear_f32_on_stream(const float* input, const uint8_t* weight, const uint8_t* scales, float* output,
                                                           uint32_t batch_rows, uint32_t rows, uint32_t cols, cudaStream_t stream) {
    return launch_block_fp8<uint8_t>(input, weight, scales, output, batch_rows, rows, cols, stream);
}

cudaError_t infer_block_fp8_f32_scale_linear_f32_on_stream(const float* input, const uint8_t* weight, const float* scales, float* output,
                                                           uint32_t batch_rows, uint32_t rows, uint32_t cols, cudaStream_t stream) {
    return launch_block_fp8<float>(input, weight, scales, output, batch_rows, rows, cols, stream);
}

}  // extern "C"
