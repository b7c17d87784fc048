// Activation / weight quantizers: NVFP4 (E2M1 codes + UE4M3 block scales) and FP8 E4M3.
//
// HBM-bound element-wise work: one CTA per row, each thread owns whole 16-element blocks so the
// block maximum, the scale byte and the eight packed bytes are produced without shuffles, loads
// are 128-bit and the packed store is one 64-bit word per block.
//
// Numerics restate crates/eider-cuda/native/non_gemm.cu:106-155 with IEEE divisions
// (the reference's host twin, crates/eider-cuda/src/format.rs:242-292, is the arbiter).
#include "common.cuh"
#include "rowops.cuh"
#include "eider_b200.h"

namespace eider {

namespace {

template <typename T> struct Loader;
template <> struct Loader<float> {
    static __device__ __forceinline__ void load16(const float* p, float (&v)[16]) {
        const float4* q = reinterpret_cast<const float4*>(p);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float4 f = __ldg(q + i);
            v[4 * i] = f.x; v[4 * i + 1] = f.y; v[4 * i + 2] = f.z; v[4 * i + 3] = f.w;
        }
    }
    static __device__ __forceinline__ float load1(const float* p) { return __ldg(p); }
};
template <> struct Loader<uint16_t> {
    static __device__ __forceinline__ void load16(const uint16_t* p, float (&v)[16]) {
        const uint4* q = reinterpret_cast<const uint4*>(p);
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            uint4 u = __ldg(q + i);
            uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                v[8 * i + 2 * j] = __uint_as_float(w[j] << 16);
                v[8 * i + 2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
            }
        }
    }
    static __device__ __forceinline__ float load1(const uint16_t* p) { return bf16_bits_to_float(__ldg(p)); }
};

template <typename T>
__device__ __forceinline__ void load_block(const T* row, uint32_t k, uint32_t b, bool vec_ok, float (&v)[16],
                                           uint32_t& valid) {
    uint32_t start = b * 16;
    valid = min(16u, k - start);
    if (valid == 16 && vec_ok) {
        Loader<T>::load16(row + start, v);
    } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) v[i] = static_cast<uint32_t>(i) < valid ? Loader<T>::load1(row + start + i) : 0.0f;
    }
}

__device__ __forceinline__ float block_max(float v, float* smem) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    if ((threadIdx.x & 31) == 0) smem[threadIdx.x >> 5] = v;
    __syncthreads();
    float r = smem[0];
    for (uint32_t w = 1; w < (blockDim.x >> 5); ++w) r = fmaxf(r, smem[w]);
    __syncthreads();
    return r;
}

enum ScaleMode { kStatic = 0, kPerRow = 1 };

// Eight consecutive elements of a row (half a 16-element block) per thread: 128-bit loads, the block maximum
// is completed with one shuffle between the two lanes of a block, one 32-bit packed store per thread.
template <typename T> struct Half8;
template <> struct Half8<float> {
    static __device__ __forceinline__ void load(const float* p, float (&v)[8]) {
        const float4 a = __ldg(reinterpret_cast<const float4*>(p));
        const float4 b = __ldg(reinterpret_cast<const float4*>(p) + 1);
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    }
};
template <> struct Half8<uint16_t> {
    static __device__ __forceinline__ void load(const uint16_t* p, float (&v)[8]) {
        const uint4 u = __ldg(reinterpret_cast<const uint4*>(p));
        const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            v[2 * j] = __uint_as_float(w[j] << 16);
            v[2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
        }
    }
};

// One CTA per row, one thread per 8 elements (rows longer than 8 * blockDim are walked in passes).  Requires
// K % 16 == 0 and 16-byte aligned rows; the generic kernel below takes everything else.
// TILED: scales go to the 128x4 tile layout with outer = row (activations); otherwise row-major [rows][K/16].
template <typename T, int MODE, bool TILED, int PASSES>
__global__ void __launch_bounds__(1024) quantize_nvfp4_fast_kernel(const T* __restrict__ input, uint8_t* __restrict__ packed,
                                                                   uint8_t* __restrict__ scales,
                                                                   float* __restrict__ row_scales, uint32_t rows, uint32_t k,
                                                                   float input_scale) {
    __shared__ float red[32];
    // a GEMM launched behind this kernel may begin its prologue right away (it waits for this grid before it reads)
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const uint32_t row = blockIdx.x;
    const T* src = input + static_cast<size_t>(row) * k;
    const uint32_t halves = k / 8;
    float held[PASSES][8];
#pragma unroll
    for (int j = 0; j < PASSES; ++j) {
        const uint32_t h = threadIdx.x + j * blockDim.x;
        if (h < halves) {
            Half8<T>::load(src + h * 8, held[j]);
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) held[j][i] = 0.0f;
        }
    }
    float g = input_scale;
    if (MODE == kPerRow) {
        float amax = 0.0f;
#pragma unroll
        for (int j = 0; j < PASSES; ++j)
#pragma unroll
            for (int i = 0; i < 8; ++i) amax = fmaxf(amax, finite_abs(held[j][i]));
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
        __syncthreads();
        amax = red[0];
        for (uint32_t w = 1; w < (blockDim.x >> 5); ++w) amax = fmaxf(amax, red[w]);
        g = row_scale_pow2(amax);
        if (threadIdx.x == 0) row_scales[row] = g;
    }
    const Divisor dg = make_divisor(g);
    const bool unit = g == 1.0f;  // (x / 1 is x: the usual case of the routed-MoE rows and of calibrated scales folded elsewhere)
    uint8_t* prow = packed + static_cast<size_t>(row) * (k / 2);
    const uint32_t blocks = k / 16;
#pragma unroll
    for (int j = 0; j < PASSES; ++j) {
        const uint32_t h = threadIdx.x + j * blockDim.x;
        float v[8];
        float amax = 0.0f;
        // one max per element: fmaxf drops NaNs as the quantizer's maximum does; an infinity (which it must drop too) shows
        // in the result and sends the whole warp down the careful path for this pass
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            v[i] = unit ? held[j][i] : div_rn(held[j][i], dg);
            amax = fmaxf(amax, fabsf(v[i]));
        }
        const bool careful = __any_sync(0xffffffffu, amax == __int_as_float(0x7f800000));
        if (careful) {
            amax = 0.0f;
#pragma unroll
            for (int i = 0; i < 8; ++i) amax = fmaxf(amax, finite_abs(v[i]));
        }
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));  // the other half of the block (all lanes take part)
        if (h >= halves) continue;
        const uint8_t sc = amax == 0.0f ? 0 : ue4m3_code(div6_rn(amax));
        const float sv = e4m3_value(sc);
        const Divisor ds = make_divisor(sv == 0.0f ? 1.0f : sv);
        uint32_t w = 0;
        if (sv == 0.0f) {
            // an all-zero (or all non-finite) block: zero codes
        } else if (!careful) {
#pragma unroll
            for (int i = 0; i < 8; i += 2)
                w |= static_cast<uint32_t>(e2m1x2_code(div_rn_finite(v[i], ds), div_rn_finite(v[i + 1], ds))) << (i * 4);
        } else {
#pragma unroll
            for (int i = 0; i < 8; i += 2)
                w |= static_cast<uint32_t>(e2m1x2_code(div_rn(v[i], ds), div_rn(v[i + 1], ds))) << (i * 4);
        }
        *reinterpret_cast<uint32_t*>(prow + h * 4) = w;
        if ((h & 1) == 0) {
            const uint32_t b = h >> 1;
            if (TILED) scales[tiled_scale_offset(row, b, k)] = sc;
            else scales[static_cast<size_t>(row) * blocks + b] = sc;
        }
    }
}

// Per-row-scale quantizer of the prefill GEMM: one CTA per row, one thread per 16-element block, the whole grid
// resident in one wave.  With the power-of-two row scale the first division is an exact multiply, the block maximum
// needs no shuffle, and the scale byte, its reciprocal and the tile offset are computed once per 16 elements.
template <typename T, bool TILED>
__global__ void __launch_bounds__(1024) quantize_nvfp4_rowscale_kernel(const T* __restrict__ input, uint8_t* __restrict__ packed,
                                                                       uint8_t* __restrict__ scales,
                                                                       float* __restrict__ row_scales, uint32_t k) {
    __shared__ float red[32];
    __shared__ float row_amax;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const uint32_t row = blockIdx.x;
    const uint32_t blocks = k / 16;
    const uint32_t b = threadIdx.x;
    float v[16];
    float amax = 0.0f;
    bool has_inf = false;
    if (b < blocks) {
        Loader<T>::load16(input + static_cast<size_t>(row) * k + b * 16, v);
        // one max per element: fmaxf drops NaNs as the quantizer's maximum does; an infinity (which it must drop too) shows
        // in the result and sends the block down the careful path
#pragma unroll
        for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(v[i]));
        has_inf = amax == __int_as_float(0x7f800000);
        if (has_inf) {
            amax = 0.0f;
#pragma unroll
            for (int i = 0; i < 16; ++i) amax = fmaxf(amax, finite_abs(v[i]));
        }
    }
    float bmax = amax;  // maximum of this thread's block, before scaling
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
    __syncthreads();
    if (threadIdx.x < 32) {
        float m = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.0f;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        if (threadIdx.x == 0) row_amax = m;
    }
    __syncthreads();
    const float g = row_scale_pow2(row_amax);
    if (threadIdx.x == 0) row_scales[row] = g;
    if (b >= blocks) return;
    const float inv_g = pow2_reciprocal(g);
    bmax *= inv_g;  // exact: scaling by a power of two commutes with the maximum
    const uint8_t sc = bmax == 0.0f ? 0 : ue4m3_code(div6_rn(bmax));
    const float sv = e4m3_value(sc);
    const Divisor ds = make_divisor(sv == 0.0f ? 1.0f : sv);
    uint32_t w[2] = {0u, 0u};
    if (sv == 0.0f) {
        // an all-zero (or all non-finite) block: zero codes
    } else if (!has_inf && ds.fast) {
#pragma unroll
        for (int i = 0; i < 16; i += 2)
            w[i / 8] |= static_cast<uint32_t>(e2m1x2_code(div_rn_finite(v[i] * inv_g, ds), div_rn_finite(v[i + 1] * inv_g, ds))) << ((i % 8) * 4);
    } else {
#pragma unroll
        for (int i = 0; i < 16; i += 2)
            w[i / 8] |= static_cast<uint32_t>(e2m1x2_code(div_rn(v[i] * inv_g, ds), div_rn(v[i + 1] * inv_g, ds))) << ((i % 8) * 4);
    }
    *reinterpret_cast<uint2*>(packed + static_cast<size_t>(row) * (k / 2) + b * 8) = make_uint2(w[0], w[1]);
    if (TILED) scales[tiled_scale_offset(row, b, k)] = sc;
    else scales[static_cast<size_t>(row) * blocks + b] = sc;
}

// Generic kernel: any K (ragged last block, odd K) and any alignment.  One CTA per row, one thread per block.
template <typename T, int MODE, bool TILED>
__global__ void __launch_bounds__(256) quantize_nvfp4_kernel(const T* __restrict__ input, uint8_t* __restrict__ packed,
                                                             uint8_t* __restrict__ scales, float* __restrict__ row_scales,
                                                             uint32_t rows, uint32_t k, float input_scale) {
    __shared__ float red[8];
    const uint32_t row = blockIdx.x;
    const T* src = input + static_cast<size_t>(row) * k;
    const uint32_t blocks = (k + 15) / 16;
    const bool vec_ok = (k % 16 == 0) && ((reinterpret_cast<uintptr_t>(input) & 15) == 0);
    float g = input_scale;
    if (MODE == kPerRow) {
        float amax = 0.0f;
        for (uint32_t b = threadIdx.x; b < blocks; b += blockDim.x) {
            float v[16];
            uint32_t valid;
            load_block(src, k, b, vec_ok, v, valid);
#pragma unroll
            for (int i = 0; i < 16; ++i)
                if (isfinite(v[i])) amax = fmaxf(amax, fabsf(v[i]));
        }
        amax = block_max(amax, red);
        g = row_scale_pow2(amax);
        if (threadIdx.x == 0) row_scales[row] = g;
    }
    const Divisor dg = make_divisor(g);
    uint8_t* prow = packed + static_cast<size_t>(row) * (k / 2);
    for (uint32_t b = threadIdx.x; b < blocks; b += blockDim.x) {
        float v[16];
        uint32_t valid;
        load_block(src, k, b, vec_ok, v, valid);
#pragma unroll
        for (int i = 0; i < 16; ++i) v[i] = div_rn(v[i], dg);
        uint2 bytes;
        uint8_t sc = quantize_block16(v, valid, &bytes);
        if (valid == 16 && (k % 16 == 0)) {
            *reinterpret_cast<uint2*>(prow + b * 8) = bytes;
        } else {
            // ragged tail: element (row*k + i) lives in nibble (row*k + i) & 1 of byte (row*k + i) / 2
            uint32_t w[2] = {bytes.x, bytes.y};
            for (uint32_t i = 0; i < valid; ++i) {
                size_t flat = static_cast<size_t>(row) * k + b * 16 + i;
                uint32_t code = (w[i / 8] >> ((i % 8) * 4)) & 0xfu;
                uint8_t* dst = packed + flat / 2;
                if (flat & 1) *dst = static_cast<uint8_t>((*dst & 0x0f) | (code << 4));
                else *dst = static_cast<uint8_t>((*dst & 0xf0) | code);
            }
        }
        if (TILED) scales[tiled_scale_offset(row, b, k)] = sc;
        else scales[static_cast<size_t>(row) * blocks + b] = sc;
    }
}

template <typename T, int MODE, bool TILED>
cudaError_t launch_quantize_nvfp4(const T* input, uint8_t* packed, uint8_t* scales, float* row_scales, uint32_t rows,
                                  uint32_t k, float input_scale, cudaStream_t stream) {
    const bool aligned = (k % 16 == 0) && ((reinterpret_cast<uintptr_t>(input) & 15) == 0) &&
                         ((reinterpret_cast<uintptr_t>(packed) & 3) == 0);
    const uint32_t halves = k / 8;
    if (MODE == kPerRow && aligned && k / 16 <= 1024 && (reinterpret_cast<uintptr_t>(packed) & 7) == 0) {
        const uint32_t threads = (k / 16 + 31) / 32 * 32;
        quantize_nvfp4_rowscale_kernel<T, TILED><<<rows, threads, 0, stream>>>(input, packed, scales, row_scales, k);
        return cudaGetLastError();
    }
    if (aligned && halves <= 4096) {
        // an even number of threads, a multiple of 32, so both halves of a block sit in one warp
        const uint32_t passes = (halves + 1023) / 1024;
        uint32_t threads = ((halves + passes - 1) / passes + 31) / 32 * 32;
        switch (passes) {
            case 1: quantize_nvfp4_fast_kernel<T, MODE, TILED, 1><<<rows, threads, 0, stream>>>(input, packed, scales, row_scales, rows, k, input_scale); break;
            case 2: quantize_nvfp4_fast_kernel<T, MODE, TILED, 2><<<rows, threads, 0, stream>>>(input, packed, scales, row_scales, rows, k, input_scale); break;
            case 3: quantize_nvfp4_fast_kernel<T, MODE, TILED, 3><<<rows, threads, 0, stream>>>(input, packed, scales, row_scales, rows, k, input_scale); break;
            default: quantize_nvfp4_fast_kernel<T, MODE, TILED, 4><<<rows, threads, 0, stream>>>(input, packed, scales, row_scales, rows, k, input_scale); break;
        }
        return cudaGetLastError();
    }
    quantize_nvfp4_kernel<T, MODE, TILED><<<rows, 256, 0, stream>>>(input, packed, scales, row_scales, rows, k, input_scale);
    return cudaGetLastError();
}

// Residual NVFP4 expansion of a few activation rows for the tensor-core decode GEMV.
//
// x ~= sum_j g_j * deq(q_j): term 0 is the ordinary NVFP4 quantization of x with the per-row scale
// g_0 = amax / 2688; every further term quantizes what the previous ones left over, with g_j = g_0 / 4^j
// (the leftover of a block is at most about 1/6 of its maximum, so the block scales stay inside E4M3).
// Eight terms carry an fp32 activation to better than 2^-17 of the row maximum, so a W4A4 block-scaled MMA
// over the expanded rows reproduces the W4A16 product (the reference keeps up to two such residual terms for
// its own W4A4 decode, crates/eider-cuda/native/sm12x_mma.cu:717-880).
// Output rows are token-major: row = token * TERMS + j; scales are tiled with outer = that row.
constexpr uint32_t kExpandThreads = 128;                     // one thread per 8 elements of the CTA's chunk
constexpr uint32_t kExpandChunk = kExpandThreads * 8;        // elements per CTA

__device__ __forceinline__ float decode_e4m3_fast(uint8_t code) {
    const __half2_raw h = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(code), __NV_E4M3);
    return __half2float(__half(__half_raw{h.x}));
}
__device__ __forceinline__ float2 decode_e2m1x2_fast(uint32_t byte) {
    const __half2_raw h = __nv_cvt_fp4x2_to_halfraw2(static_cast<__nv_fp4x2_storage_t>(byte), __NV_E2M1);
    return make_float2(__half2float(__half(__half_raw{h.x})), __half2float(__half(__half_raw{h.y})));
}

// grid = (chunks per row, tokens).  Every CTA finds the row maximum itself (the row is a few kilobytes and shared
// through L2) and then expands only its 1024-element chunk, so a handful of tokens still spreads over many SMs; the
// residual chain of a thread never leaves its registers.
template <typename T>
__global__ void __launch_bounds__(kExpandThreads) expand_nvfp4_terms_kernel(const T* __restrict__ input, uint8_t* __restrict__ packed,
                                                                            uint8_t* __restrict__ scales, float* __restrict__ col_scale,
                                                                            uint32_t k, uint32_t terms, uint32_t operand_cols) {
    __shared__ float red[kExpandThreads / 32];
    // launched as a programmatic dependent launch: the kernel after this one may start its own prologue now, and this one
    // touches memory only after the kernel before it has finished
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const uint32_t token = blockIdx.y;
    const T* src = input + static_cast<size_t>(token) * k;
    const uint32_t halves = k / 8;
    float amax = 0.0f;
    for (uint32_t h = threadIdx.x; h < halves; h += kExpandThreads) {
        float t[8];
        Half8<T>::load(src + h * 8, t);
#pragma unroll
        for (int i = 0; i < 8; ++i) amax = fmaxf(amax, finite_abs(t[i]));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
    __syncthreads();
    amax = red[0];
#pragma unroll
    for (uint32_t w = 1; w < kExpandThreads / 32; ++w) amax = fmaxf(amax, red[w]);
    float g = row_scale_pow2(amax);
    float inv_g = pow2_reciprocal(g);

    const uint32_t h = blockIdx.x * kExpandThreads + threadIdx.x;
    float r[8];
    if (h < halves) {
        Half8<T>::load(src + h * 8, r);
#pragma unroll
        for (int i = 0; i < 8; ++i)
            if (!isfinite(r[i])) r[i] = 0.0f;  // non-finite activations carry no information for a GEMV
    } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) r[i] = 0.0f;
    }
    for (uint32_t term = 0; term < terms; ++term) {
        const uint32_t row = token * terms + term;
        if (blockIdx.x == 0 && threadIdx.x == 0) col_scale[row] = g;
        float v[8];
        float bmax = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            v[i] = r[i] * inv_g;  // exact: g is a power of two
            bmax = fmaxf(bmax, fabsf(v[i]));
        }
        bmax = fmaxf(bmax, __shfl_xor_sync(0xffffffffu, bmax, 1));  // the other half of the 16-element block
        const uint8_t sc = bmax == 0.0f ? 0 : ue4m3_code(div6_rn(bmax));
        const float sv = decode_e4m3_fast(sc);
        const Divisor ds = make_divisor(sv == 0.0f ? 1.0f : sv);
        const float back = sv * g;
        uint32_t w = 0;
#pragma unroll
        for (int i = 0; i < 8; i += 2) {
            const float lo = sv == 0.0f ? 0.0f : div_rn(v[i], ds);
            const float hi = sv == 0.0f ? 0.0f : div_rn(v[i + 1], ds);
            const uint32_t byte = e2m1x2_code(lo, hi);
            w |= byte << (i * 4);
            const float2 q = decode_e2m1x2_fast(byte);  // leftover for the next term
            r[i] = fmaf(-q.x, back, r[i]);
            r[i + 1] = fmaf(-q.y, back, r[i + 1]);
        }
        if (h < halves) {
            *reinterpret_cast<uint32_t*>(packed + static_cast<size_t>(row) * (k / 2) + h * 4) = w;
            // scale bytes: the 128 x 4 tiles of a GEMM operand, or (operand_cols != 0) the layout the single-launch decode
            // kernel copies straight into shared memory: [64-element block][operand row][16 bytes], first four used
            if ((h & 1) == 0)
                scales[operand_cols ? ((static_cast<size_t>(h >> 3) * operand_cols + row) * 16 + ((h >> 1) & 3))
                                    : tiled_scale_offset(row, h >> 1, k)] = sc;
        }
        g *= 0.25f;
        inv_g *= 4.0f;
    }
}

// Fused SiLU(gate) * up -> NVFP4 quantize (crates/eider-cuda/native/non_gemm.cu:559-629): the producer in front of the
// down projection without the fp32 round trip.  gate = row[0..k), up = row[k..2k), sigmoid = 1 / (1 + expf(-g)),
// value = (g * sigmoid * up) / input_scale in that order, then the block quantizer.  One thread per 16-element block,
// grid = (blocks of 256 threads, tokens); k is a multiple of 16 and rows are 16-byte aligned on this path.
__global__ void __launch_bounds__(256) silu_mul_quantize_nvfp4_kernel(const float* __restrict__ gate_up, uint8_t* __restrict__ packed,
                                                                      uint8_t* __restrict__ scales, uint32_t k, float input_scale) {
    const uint32_t token = blockIdx.y;
    const uint32_t b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= k / 16) return;
    const float* gate = gate_up + static_cast<size_t>(token) * 2 * k + b * 16;
    const float* up = gate + k;
    const Divisor di = make_divisor(input_scale);
    float v[16];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        const float4 g4 = __ldg(reinterpret_cast<const float4*>(gate) + q);
        const float4 u4 = __ldg(reinterpret_cast<const float4*>(up) + q);
        const float g[4] = {g4.x, g4.y, g4.z, g4.w}, u[4] = {u4.x, u4.y, u4.z, u4.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            v[4 * q + i] = div_rn(rowops::silu_sigmoid_mul(g[i], u[i]), di);
        }
    }
    uint2 bytes;
    const uint8_t sc = quantize_block16(v, 16, &bytes);
    *reinterpret_cast<uint2*>(packed + static_cast<size_t>(token) * (k / 2) + b * 8) = bytes;
    scales[tiled_scale_offset(token, b, k)] = sc;
}

// Fused RMSNorm -> NVFP4 quantize (crates/eider-cuda/native/non_gemm.cu:193-288): one CTA per row.  Pass one sums the
// squares (per-thread strided partial sums, warp shuffles, then the warp sums in warp order: a fixed order for a given
// launch shape), pass two gives every thread 16-element blocks: value = x * inverse_rms * weight / input_scale in that
// order, then the block quantizer.  The row is read twice; the second read hits L1/L2.
// PAIR (non_gemm.cu:290-419): a second NVFP4 term holds what the first left, residual = value - e2m1(code) * scale (one
// FMA), quantized per block with its own scale byte.
template <bool PAIR>
__global__ void __launch_bounds__(256) rms_norm_quantize_nvfp4_kernel(const float* __restrict__ input, const float* __restrict__ weight,
                                                                      uint8_t* __restrict__ packed, uint8_t* __restrict__ scales,
                                                                      uint8_t* __restrict__ residual_packed,
                                                                      uint8_t* __restrict__ residual_scales, uint32_t cols, float eps,
                                                                      float input_scale) {
    __shared__ float red[8];
    const uint32_t row = blockIdx.x;
    const float* x = input + static_cast<size_t>(row) * cols;
    const float inv = rowops::inverse_rms(rowops::block_sum_ordered(rowops::thread_sum_squares_f4(x, cols), red), cols, eps);
    const Divisor di = make_divisor(input_scale);
    for (uint32_t b = threadIdx.x; b < cols / 16; b += blockDim.x) {
        float v[16];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const float4 x4 = __ldg(reinterpret_cast<const float4*>(x + b * 16) + q);
            const float4 w4 = __ldg(reinterpret_cast<const float4*>(weight + b * 16) + q);
            v[4 * q + 0] = div_rn(rowops::normed(x4.x, inv, w4.x), di);
            v[4 * q + 1] = div_rn(rowops::normed(x4.y, inv, w4.y), di);
            v[4 * q + 2] = div_rn(rowops::normed(x4.z, inv, w4.z), di);
            v[4 * q + 3] = div_rn(rowops::normed(x4.w, inv, w4.w), di);
        }
        uint2 bytes;
        const uint8_t sc = quantize_block16(v, 16, &bytes);
        *reinterpret_cast<uint2*>(packed + static_cast<size_t>(row) * (cols / 2) + b * 8) = bytes;
        scales[tiled_scale_offset(row, b, cols)] = sc;
        if (PAIR) {
            const float sv = e4m3_value(sc);
            const uint32_t w[2] = {bytes.x, bytes.y};
#pragma unroll
            for (int i = 0; i < 16; ++i) v[i] = fmaf(-e2m1_value((w[i / 8] >> ((i % 8) * 4)) & 0xfu), sv, v[i]);
            const uint8_t rsc = quantize_block16(v, 16, &bytes);
            *reinterpret_cast<uint2*>(residual_packed + static_cast<size_t>(row) * (cols / 2) + b * 8) = bytes;
            residual_scales[tiled_scale_offset(row, b, cols)] = rsc;
        }
    }
}

// Post-norm residual add + quantizing pre-norm in one kernel (crates/eider-cuda/native/non_gemm.cu:746-870): one CTA per
// row; h = input * inverse_rms0 * input_weight + residual is written to `output`, kept in shared memory and squared for
// the second norm, then the RMSNorm quantizer runs on the staged row.  Sums run in the same fixed order as above.
__global__ void __launch_bounds__(256) rms_norm_add_rms_norm_quantize_nvfp4_kernel(
    const float* __restrict__ input, const float* __restrict__ input_weight, const float* __restrict__ residual,
    float* __restrict__ output, const float* __restrict__ quant_weight, uint8_t* __restrict__ packed, uint8_t* __restrict__ scales,
    uint32_t cols, float input_eps, float quant_eps, float input_scale) {
    extern __shared__ __align__(16) float staged[];
    __shared__ float red[8];
    const uint32_t row = blockIdx.x;
    const size_t off = static_cast<size_t>(row) * cols;
    const float inv0 = rowops::inverse_rms(rowops::block_sum_ordered(rowops::thread_sum_squares_f4(input + off, cols), red), cols, input_eps);
    float ss2 = 0.0f;
    for (uint32_t i = threadIdx.x; i < cols / 4; i += blockDim.x) {
        const float4 v = __ldg(reinterpret_cast<const float4*>(input + off) + i);
        const float4 w = __ldg(reinterpret_cast<const float4*>(input_weight) + i);
        const float4 r = __ldg(reinterpret_cast<const float4*>(residual + off) + i);
        float4 h;
        h.x = rowops::normed_add(v.x, inv0, w.x, r.x);
        h.y = rowops::normed_add(v.y, inv0, w.y, r.y);
        h.z = rowops::normed_add(v.z, inv0, w.z, r.z);
        h.w = rowops::normed_add(v.w, inv0, w.w, r.w);
        reinterpret_cast<float4*>(output + off)[i] = h;
        reinterpret_cast<float4*>(staged)[i] = h;
        ss2 = fmaf(h.x, h.x, ss2); ss2 = fmaf(h.y, h.y, ss2); ss2 = fmaf(h.z, h.z, ss2); ss2 = fmaf(h.w, h.w, ss2);
    }
    const float inv1 = rowops::inverse_rms(rowops::block_sum_ordered(ss2, red), cols, quant_eps);  // (its barriers order the staging)
    const Divisor di = make_divisor(input_scale);
    for (uint32_t b = threadIdx.x; b < cols / 16; b += blockDim.x) {
        float v[16];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const float4 h4 = reinterpret_cast<const float4*>(staged + b * 16)[q];
            const float4 w4 = __ldg(reinterpret_cast<const float4*>(quant_weight + b * 16) + q);
            v[4 * q + 0] = div_rn(rowops::normed(h4.x, inv1, w4.x), di);
            v[4 * q + 1] = div_rn(rowops::normed(h4.y, inv1, w4.y), di);
            v[4 * q + 2] = div_rn(rowops::normed(h4.z, inv1, w4.z), di);
            v[4 * q + 3] = div_rn(rowops::normed(h4.w, inv1, w4.w), di);
        }
        uint2 bytes;
        const uint8_t sc = quantize_block16(v, 16, &bytes);
        *reinterpret_cast<uint2*>(packed + static_cast<size_t>(row) * (cols / 2) + b * 8) = bytes;
        scales[tiled_scale_offset(row, b, cols)] = sc;
    }
}

// Per-token dynamic FP8: s = amax / 448 (1 when 0), q = e4m3(x / s)
// (crates/eider-cuda/native/non_gemm.cu:9952-9974, 10028-10066).
template <typename T, bool DYNAMIC>
__global__ void __launch_bounds__(256) quantize_fp8_kernel(const T* __restrict__ input, uint8_t* __restrict__ q,
                                                           float* __restrict__ row_scale, uint32_t rows, uint32_t cols,
                                                           float static_scale) {
    __shared__ float red[8];
    if (DYNAMIC) {
        // (the dynamic quantizers are launched as programmatic dependent launches: the kernel after this one may start its
        // prologue now, and this one touches memory only after the kernel before it has finished)
        asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
        asm volatile("griddepcontrol.wait;" ::: "memory");
    }
    const uint32_t row = blockIdx.x;
    const T* src = input + static_cast<size_t>(row) * cols;
    float s = static_scale;
    const bool vec_ok = (cols % 16 == 0) && ((reinterpret_cast<uintptr_t>(input) & 15) == 0) &&
                        ((reinterpret_cast<uintptr_t>(q) & 15) == 0);
    if (DYNAMIC) {
        float amax = 0.0f;
        if (vec_ok) {
            for (uint32_t b = threadIdx.x; b < cols / 16; b += blockDim.x) {
                float v[16];
                Loader<T>::load16(src + b * 16, v);
#pragma unroll
                for (int i = 0; i < 16; ++i)
                    if (isfinite(v[i])) amax = fmaxf(amax, fabsf(v[i]));
            }
        } else {
            for (uint32_t i = threadIdx.x; i < cols; i += blockDim.x) {
                float v = Loader<T>::load1(src + i);
                if (isfinite(v)) amax = fmaxf(amax, fabsf(v));
            }
        }
        amax = block_max(amax, red);
        s = amax == 0.0f ? 1.0f : __fdiv_rn(amax, 448.0f);
        if (threadIdx.x == 0) row_scale[row] = s;
    }
    uint8_t* dst = q + static_cast<size_t>(row) * cols;
    if (vec_ok) {
        for (uint32_t b = threadIdx.x; b < cols / 16; b += blockDim.x) {
            float v[16];
            Loader<T>::load16(src + b * 16, v);
            uint32_t w[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                w[j] = 0;
#pragma unroll
                for (int i = 0; i < 4; ++i) w[j] |= static_cast<uint32_t>(e4m3_satfinite(__fdiv_rn(v[4 * j + i], s))) << (8 * i);
            }
            *reinterpret_cast<uint4*>(dst + b * 16) = make_uint4(w[0], w[1], w[2], w[3]);
        }
    } else {
        for (uint32_t i = threadIdx.x; i < cols; i += blockDim.x) dst[i] = e4m3_satfinite(__fdiv_rn(Loader<T>::load1(src + i), s));
    }
}

// Row-major [N][K/16] scale bytes -> 128x4 tiled layout (crates/eider-format/src/modelopt.rs:1148-1161).
__global__ void scales_to_tiled_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, uint32_t rows,
                                       uint32_t k) {
    const uint32_t blocks = k / 16;
    size_t total = static_cast<size_t>(rows) * blocks;
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        uint32_t r = static_cast<uint32_t>(i / blocks), b = static_cast<uint32_t>(i % blocks);
        dst[tiled_scale_offset(r, b, k)] = src[i];
    }
}

bool bad_scale(float s) { return !(s > 0.0f) || !isfinite(s); }

template <typename Kernel, typename T>
cudaError_t launch_dynamic_fp8(Kernel kernel, const T* input, uint8_t* q, float* row_scale, uint32_t rows, uint32_t cols, cudaStream_t stream) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(rows);
    cfg.blockDim = dim3(256);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, input, q, row_scale, rows, cols, 1.0f);
}

}  // namespace

// Launcher shared with the decode plan's operand object (scale bytes in the tiled GEMM layout or, operand_cols = 16 / 32, in
// the decode kernel's operand layout).
cudaError_t expand_nvfp4_terms_launch(const void* input, int input_is_bf16, uint8_t* packed, uint8_t* scales, float* col_scale,
                                      uint32_t tokens, uint32_t in_features, uint32_t terms, uint32_t operand_cols, cudaStream_t stream) {
    if (!input || !packed || !scales || !col_scale || tokens == 0 || in_features == 0 || in_features % 16 != 0 ||
        terms == 0 || terms > 16 || in_features / 8 > 4096 || (reinterpret_cast<uintptr_t>(input) & 15) != 0)
        return cudaErrorInvalidValue;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((in_features + kExpandChunk - 1) / kExpandChunk, tokens);
    cfg.blockDim = dim3(kExpandThreads);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (input_is_bf16)
        return cudaLaunchKernelEx(&cfg, expand_nvfp4_terms_kernel<uint16_t>, static_cast<const uint16_t*>(input), packed, scales,
                                  col_scale, in_features, terms, operand_cols);
    return cudaLaunchKernelEx(&cfg, expand_nvfp4_terms_kernel<float>, static_cast<const float*>(input), packed, scales, col_scale,
                              in_features, terms, operand_cols);
}

}  // namespace eider

using namespace eider;

extern "C" {

cudaError_t infer_quantize_nvfp4_col_major_f32_on_stream(const float* input, uint8_t* packed, uint8_t* scales,
                                                         uint32_t rows, uint32_t cols, float input_scale,
                                                         cudaStream_t stream) {
    if (!input || !packed || !scales || rows == 0 || cols == 0 || bad_scale(input_scale)) return cudaErrorInvalidValue;
    return launch_quantize_nvfp4<float, kStatic, true>(input, packed, scales, nullptr, cols, rows, input_scale, stream);
}

cudaError_t infer_quantize_nvfp4_col_major_f32(const float* input, uint8_t* packed, uint8_t* scales, uint32_t rows,
                                               uint32_t cols, float input_scale) {
    return infer_quantize_nvfp4_col_major_f32_on_stream(input, packed, scales, rows, cols, input_scale, nullptr);
}

cudaError_t eider_b200_quantize_nvfp4_bf16_on_stream(const uint16_t* input, uint8_t* packed, uint8_t* scales,
                                                     uint32_t rows, uint32_t cols, float input_scale,
                                                     cudaStream_t stream) {
    if (!input || !packed || !scales || rows == 0 || cols == 0 || bad_scale(input_scale)) return cudaErrorInvalidValue;
    return launch_quantize_nvfp4<uint16_t, kStatic, true>(input, packed, scales, nullptr, cols, rows, input_scale, stream);
}

cudaError_t eider_b200_quantize_nvfp4_rowscale_on_stream(const void* input, int input_is_bf16, uint8_t* packed,
                                                         uint8_t* scales, float* row_scales, uint32_t rows,
                                                         uint32_t cols, cudaStream_t stream) {
    if (!input || !packed || !scales || !row_scales || rows == 0 || cols == 0) return cudaErrorInvalidValue;
    if (input_is_bf16)
        return launch_quantize_nvfp4<uint16_t, kPerRow, true>(static_cast<const uint16_t*>(input), packed, scales, row_scales,
                                                              cols, rows, 1.0f, stream);
    return launch_quantize_nvfp4<float, kPerRow, true>(static_cast<const float*>(input), packed, scales, row_scales, cols,
                                                       rows, 1.0f, stream);
}

cudaError_t eider_b200_quantize_nvfp4_weight_on_stream(const void* weight, int input_is_bf16, uint8_t* packed,
                                                       uint8_t* scales_row_major, uint32_t out_features,
                                                       uint32_t in_features, float global_scale, cudaStream_t stream) {
    if (!weight || !packed || !scales_row_major || out_features == 0 || in_features == 0 || in_features % 16 != 0 ||
        bad_scale(global_scale))
        return cudaErrorInvalidValue;
    if (input_is_bf16)
        return launch_quantize_nvfp4<uint16_t, kStatic, false>(static_cast<const uint16_t*>(weight), packed, scales_row_major,
                                                               nullptr, out_features, in_features, global_scale, stream);
    return launch_quantize_nvfp4<float, kStatic, false>(static_cast<const float*>(weight), packed, scales_row_major, nullptr,
                                                        out_features, in_features, global_scale, stream);
}

cudaError_t eider_b200_nvfp4_scales_to_tiled_on_stream(const uint8_t* scales_row_major, uint8_t* scales_tiled,
                                                       uint32_t out_features, uint32_t in_features,
                                                       cudaStream_t stream) {
    if (!scales_row_major || !scales_tiled || out_features == 0 || in_features == 0 || in_features % 16 != 0)
        return cudaErrorInvalidValue;
    cudaError_t st = cudaMemsetAsync(scales_tiled, 0, scale_layout_len(out_features, in_features), stream);
    if (st != cudaSuccess) return st;
    size_t total = static_cast<size_t>(out_features) * (in_features / 16);
    uint32_t grid = static_cast<uint32_t>((total + 255) / 256);
    if (grid > 148 * 16) grid = 148 * 16;
    scales_to_tiled_kernel<<<grid, 256, 0, stream>>>(scales_row_major, scales_tiled, out_features, in_features);
    return cudaGetLastError();
}

size_t eider_b200_nvfp4_scale_layout_len(size_t outer, size_t inner) { return scale_layout_len(outer, inner); }

cudaError_t eider_b200_expand_nvfp4_terms_on_stream(const void* input, int input_is_bf16, uint8_t* packed,
                                                    uint8_t* scales, float* col_scale, uint32_t tokens, uint32_t in_features,
                                                    uint32_t terms, cudaStream_t stream) {
    return eider::expand_nvfp4_terms_launch(input, input_is_bf16, packed, scales, col_scale, tokens, in_features, terms, 0, stream);
}


cudaError_t infer_rms_norm_quantize_nvfp4_col_major_f32_on_stream(const float* input, const float* weight, uint8_t* packed,
                                                                  uint8_t* scales, uint32_t rows, uint32_t cols, float eps,
                                                                  float input_scale, cudaStream_t stream) {
    if (!input || !weight || !packed || !scales || rows == 0 || cols == 0 || cols % 16 != 0 || bad_scale(input_scale) ||
        ((reinterpret_cast<uintptr_t>(input) | reinterpret_cast<uintptr_t>(weight)) & 15) != 0 ||
        (reinterpret_cast<uintptr_t>(packed) & 7) != 0)
        return cudaErrorInvalidValue;
    rms_norm_quantize_nvfp4_kernel<false><<<rows, 256, 0, stream>>>(input, weight, packed, scales, nullptr, nullptr, cols, eps, input_scale);
    return cudaGetLastError();
}

cudaError_t infer_rms_norm_quantize_nvfp4_pair_col_major_f32_on_stream(const float* input, const float* weight, uint8_t* packed,
                                                                       uint8_t* scales, uint8_t* residual_packed,
                                                                       uint8_t* residual_scales, uint32_t rows, uint32_t cols,
                                                                       float eps, float input_scale, cudaStream_t stream) {
    if (!input || !weight || !packed || !scales || !residual_packed || !residual_scales || rows == 0 || cols == 0 ||
        cols % 16 != 0 || bad_scale(input_scale) ||
        ((reinterpret_cast<uintptr_t>(input) | reinterpret_cast<uintptr_t>(weight)) & 15) != 0 ||
        ((reinterpret_cast<uintptr_t>(packed) | reinterpret_cast<uintptr_t>(residual_packed)) & 7) != 0)
        return cudaErrorInvalidValue;
    rms_norm_quantize_nvfp4_kernel<true><<<rows, 256, 0, stream>>>(input, weight, packed, scales, residual_packed, residual_scales,
                                                                   cols, eps, input_scale);
    return cudaGetLastError();
}

// The row is staged in dynamic shared memory beside the kernel's 32 bytes of static shared memory; both must fit the
// 48 KB a kernel gets without opting in.
constexpr uint32_t kAddNormMaxCols = (48 * 1024 - 64) / 4 / 16 * 16;  // 12272

cudaError_t infer_rms_norm_add_then_rms_norm_quantize_nvfp4_f32_on_stream(const float* input, const float* input_weight,
                                                                          const float* residual, float* output,
                                                                          const float* quant_weight, uint8_t* packed,
                                                                          uint8_t* scales, uint32_t rows, uint32_t cols,
                                                                          float input_eps, float quant_eps, float input_scale,
                                                                          cudaStream_t stream) {
    if (!input || !input_weight || !residual || !output || !quant_weight || !packed || !scales || rows == 0 || cols == 0 ||
        cols % 16 != 0 || cols > kAddNormMaxCols || !(input_eps >= 0.0f) || !isfinite(input_eps) || !(quant_eps >= 0.0f) ||
        !isfinite(quant_eps) || bad_scale(input_scale) || (reinterpret_cast<uintptr_t>(packed) & 7) != 0 ||
        ((reinterpret_cast<uintptr_t>(input) | reinterpret_cast<uintptr_t>(input_weight) | reinterpret_cast<uintptr_t>(residual) |
          reinterpret_cast<uintptr_t>(output) | reinterpret_cast<uintptr_t>(quant_weight)) & 15) != 0)
        return cudaErrorInvalidValue;
    rms_norm_add_rms_norm_quantize_nvfp4_kernel<<<rows, 256, cols * sizeof(float), stream>>>(
        input, input_weight, residual, output, quant_weight, packed, scales, cols, input_eps, quant_eps, input_scale);
    return cudaGetLastError();
}

cudaError_t eider_b200_silu_mul_halves_quantize_nvfp4_batch_on_stream(const float* gate_up, uint8_t* packed, uint8_t* scales,
                                                                      uint32_t tokens, uint32_t rows, float input_scale,
                                                                      cudaStream_t stream) {
    if (!gate_up || !packed || !scales || tokens == 0 || rows == 0 || rows % 16 != 0 || bad_scale(input_scale) ||
        (reinterpret_cast<uintptr_t>(gate_up) & 15) != 0 || (reinterpret_cast<uintptr_t>(packed) & 7) != 0)
        return cudaErrorInvalidValue;
    const dim3 grid((rows / 16 + 255) / 256, tokens);
    silu_mul_quantize_nvfp4_kernel<<<grid, 256, 0, stream>>>(gate_up, packed, scales, rows, input_scale);
    return cudaGetLastError();
}

cudaError_t infer_silu_mul_halves_quantize_nvfp4_col_major_f32_on_stream(const float* gate_up, uint8_t* packed, uint8_t* scales,
                                                                         uint32_t rows, float input_scale, cudaStream_t stream) {
    return eider_b200_silu_mul_halves_quantize_nvfp4_batch_on_stream(gate_up, packed, scales, 1, rows, input_scale, stream);
}

cudaError_t infer_quantize_fp8_e4m3_dynamic_f32_batch_on_stream(const float* input, uint8_t* quantized_input,
                                                                float* input_scale, uint32_t rows, uint32_t cols,
                                                                cudaStream_t stream) {
    if (!input || !quantized_input || !input_scale || rows == 0 || cols == 0) return cudaErrorInvalidValue;
    return launch_dynamic_fp8(quantize_fp8_kernel<float, true>, input, quantized_input, input_scale, rows, cols, stream);
}

cudaError_t infer_quantize_fp8_e4m3_dynamic_f32_on_stream(const float* input, uint8_t* quantized_input,
                                                          float* input_scale, uint32_t cols, cudaStream_t stream) {
    return infer_quantize_fp8_e4m3_dynamic_f32_batch_on_stream(input, quantized_input, input_scale, 1, cols, stream);
}

cudaError_t eider_b200_quantize_fp8_e4m3_dynamic_bf16_batch_on_stream(const uint16_t* input, uint8_t* quantized_input,
                                                                      float* input_scale, uint32_t rows, uint32_t cols,
                                                                      cudaStream_t stream) {
    if (!input || !quantized_input || !input_scale || rows == 0 || cols == 0) return cudaErrorInvalidValue;
    return launch_dynamic_fp8(quantize_fp8_kernel<uint16_t, true>, input, quantized_input, input_scale, rows, cols, stream);
}

cudaError_t infer_quantize_fp8_e4m3_f32_on_stream(const float* input, uint8_t* output, uint32_t len, float input_scale,
                                                  cudaStream_t stream) {
    if (!input || !output || len == 0 || bad_scale(input_scale)) return cudaErrorInvalidValue;
    // one logical row split over CTAs of 4096 elements keeps 128-bit accesses aligned
    const uint32_t chunk = 4096;
    uint32_t full = len / chunk;
    if (full)
        quantize_fp8_kernel<float, false><<<full, 256, 0, stream>>>(input, output, nullptr, full, chunk, input_scale);
    if (len % chunk)
        quantize_fp8_kernel<float, false><<<1, 256, 0, stream>>>(input + static_cast<size_t>(full) * chunk,
                                                                 output + static_cast<size_t>(full) * chunk, nullptr, 1,
                                                                 len % chunk, input_scale);
    return cudaGetLastError();
}

cudaError_t eider_b200_quantize_fp8_weight_on_stream(const void* weight, int input_is_bf16, uint8_t* q,
                                                     float* channel_scale, uint32_t out_features, uint32_t in_features,
                                                     cudaStream_t stream) {
    if (!weight || !q || !channel_scale || out_features == 0 || in_features == 0) return cudaErrorInvalidValue;
    if (input_is_bf16)
        quantize_fp8_kernel<uint16_t, true><<<out_features, 256, 0, stream>>>(static_cast<const uint16_t*>(weight), q,
                                                                            channel_scale, out_features, in_features, 1.0f);
    else
        quantize_fp8_kernel<float, true><<<out_features, 256, 0, stream>>>(static_cast<const float*>(weight), q,
                                                                         channel_scale, out_features, in_features, 1.0f);
    return cudaGetLastError();
}

}  // extern "C"
