// NVFP4 W4A16 decode GEMV for one or two tokens on CUDA cores, built to run at HBM speed.
//
// y[t][n] = alpha * sum_k x[t][k] * e2m1(W[n][k]) * ue4m3(S[n][k/16])      (+ beta * c[t][n])
//
// Work split: a CTA of 8 warps owns 32 rows of one 128-row scale tile, chosen as rows {8q + w + 32s} (q = CTA's
// eighth-of-32 within the tile, w = warp, s = 0..3), because in the 128 x 4 tiled scale layout the sixteen bytes at
// (k-group, row mod 32) hold the four scales of rows r, r+32, r+64, r+96: one 16-byte load feeds the four rows a warp
// works on, and the eight warps of a CTA together consume whole 128-byte lines of scales.  N / 32 CTAs (432 for
// N = 13824) spread evenly over the SMs whatever N / 128 is.
// Streaming: every lane reads 16 bytes (32 weights = two scale blocks) of each of its warp's four rows per step, the
// next step's loads are issued before this step is computed, and the first step is requested before the activation
// is staged, so the weight stream starts with the kernel.
// Arithmetic: weights go e2m1 -> f16 with cvt.rn.f16x2.e2m1x2 (exact); the activation is held in shared memory as f16
// after an exact power-of-two scaling that puts the row maximum just under 2^15 (bf16 inputs then convert exactly
// unless they are 2^-29 of the maximum or smaller; f32 inputs are split into two f16 terms, 22 bits); products are
// accumulated with the mixed-precision fma.rn.f32.f16, which is exact in the product and rounds once per add in fp32;
// each 16-element block sum is scaled by its decoded UE4M3 scale in fp32.  Warp-shuffle reduction at the end.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>

#include "common.cuh"

namespace eider {
namespace gemv_stream {

constexpr uint32_t kWarps = 8;
constexpr uint32_t kThreads = kWarps * 32;
constexpr uint32_t kRowsPerCta = 32;

struct Params {
    const void* x;            // [tokens][k] bf16 or f32
    uint32_t tokens, n, k;
    const uint8_t* w;         // [n][k/2] packed e2m1
    const uint8_t* sf;        // tiled UE4M3 scales
    uint32_t sf_tile_stride;  // bytes between 128-row scale tiles
    void* out;                // [tokens][ld_out]
    const void* c_in;
    uint32_t ld_out;
    int out_is_bf16;
    float alpha, beta;
};

__device__ __forceinline__ uint32_t e2m1x2_to_f16x2(uint32_t byte) {
    uint32_t r;
    asm("{\n\t.reg .b8 t;\n\tcvt.u8.u32 t, %1;\n\tcvt.rn.f16x2.e2m1x2 %0, t;\n\t}" : "=r"(r) : "r"(byte));
    return r;
}
__device__ __forceinline__ uint32_t e4m3x2_to_f16x2(uint32_t two_bytes) {
    uint32_t r;
    asm("{\n\t.reg .b16 t;\n\tcvt.u16.u32 t, %1;\n\tcvt.rn.f16x2.e4m3x2 %0, t;\n\t}" : "=r"(r) : "r"(two_bytes));
    return r;
}
// acc += lo(a) * lo(b) + hi(a) * hi(b), products exact, one fp32 rounding per addition
__device__ __forceinline__ void fma2_f16(float& acc, uint32_t a, uint32_t b) {
    asm("{\n\t.reg .b16 al, ah, bl, bh;\n\t"
        "mov.b32 {al, ah}, %1;\n\t"
        "mov.b32 {bl, bh}, %2;\n\t"
        "fma.rn.f32.f16 %0, al, bl, %0;\n\t"
        "fma.rn.f32.f16 %0, ah, bh, %0;\n\t}"
        : "+f"(acc)
        : "r"(a), "r"(b));
}
__device__ __forceinline__ float f16_lo_to_f32(uint32_t h2) {
    float f;
    asm("{\n\t.reg .b16 l, h;\n\tmov.b32 {l, h}, %1;\n\tcvt.f32.f16 %0, l;\n\t}" : "=f"(f) : "r"(h2));
    return f;
}
__device__ __forceinline__ float f16_hi_to_f32(uint32_t h2) {
    float f;
    asm("{\n\t.reg .b16 l, h;\n\tmov.b32 {l, h}, %1;\n\tcvt.f32.f16 %0, h;\n\t}" : "=f"(f) : "r"(h2));
    return f;
}
__device__ __forceinline__ uint32_t pack_f16x2(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.f16x2.f32 %0, %2, %1;" : "=r"(r) : "f"(lo), "f"(hi));
    return r;
}

template <typename XT> __device__ __forceinline__ float load_x(const XT* p, uint32_t i);
template <> __device__ __forceinline__ float load_x<uint16_t>(const uint16_t* p, uint32_t i) {
    return __uint_as_float(static_cast<uint32_t>(__ldg(p + i)) << 16);
}
template <> __device__ __forceinline__ float load_x<float>(const float* p, uint32_t i) { return __ldg(p + i); }

// Shared-memory position (in f16 pairs) of elements (e, e + 1), e even: the lane that owns 16-byte weight piece
// p = e / 32 reads its four 8-element groups j = (e % 32) / 8 as 16-byte vectors, lanes side by side.
__device__ __forceinline__ uint32_t x_pair_slot(uint32_t e) {
    const uint32_t piece = e >> 5, lane = piece & 31, step = piece >> 5;
    const uint32_t j = (e & 31) >> 3, t = (e & 7) >> 1;
    return ((step * 4 + j) * 32 + lane) * 4 + t;
}

// XT: activation type.  TERMS: f16 terms per activation (1 for bf16, 2 for f32).  TOKENS: 1 or 2.
template <typename XT, int TERMS, int TOKENS>
__global__ void __launch_bounds__(kThreads) gemv_stream_kernel(const Params p) {
    extern __shared__ __align__(16) uint32_t xs[];  // [TOKENS][TERMS][steps * 512] f16 pairs, permuted, zero padded
    __shared__ float red[kWarps];
    __shared__ float inv_gain[TOKENS];
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t tile = blockIdx.x >> 2, q = blockIdx.x & 3;
    const uint32_t row32 = q * 8 + warp;                 // row index modulo 32 inside the tile
    const uint32_t row0 = tile * 128 + row32;            // the warp's rows are row0 + 32 s
    const uint32_t pieces = p.k / 32;                    // 16-byte pieces per weight row
    const uint32_t steps = (pieces + 31) / 32;
    const size_t row_bytes = p.k / 2;
    const uint8_t* sf_tile = p.sf + static_cast<size_t>(tile) * p.sf_tile_stride + row32 * 16;

    // two register buffers, named rather than indexed so that they stay in registers
    uint4 wa[4], wb[4];
    uint4 sa, sb;
    auto request = [&](uint32_t step, uint4 (&wbuf)[4], uint4& sbuf) {
        const uint32_t piece = step * 32 + lane;
        if (piece < pieces) {
#pragma unroll
            for (uint32_t s = 0; s < 4; ++s) {
                const uint32_t row = row0 + 32 * s;
                wbuf[s] = row < p.n ? __ldcs(reinterpret_cast<const uint4*>(p.w + row * row_bytes) + piece) : make_uint4(0, 0, 0, 0);
            }
            sbuf = __ldg(reinterpret_cast<const uint4*>(sf_tile + static_cast<size_t>(piece >> 1) * 512));
        } else {
#pragma unroll
            for (uint32_t s = 0; s < 4; ++s) wbuf[s] = make_uint4(0, 0, 0, 0);
            sbuf = make_uint4(0, 0, 0, 0);
        }
    };
    request(0, wa, sa);  // the weight stream starts before the activation is staged

    // ---- stage the activation: x * gain as f16 (one or two terms), permuted for conflict-free 16-byte reads
    const XT* x = static_cast<const XT*>(p.x);
    const uint32_t pairs = p.k / 2;
    const uint32_t plane = steps * 512;  // f16 pairs per (token, term), a whole number of 32-lane steps
    for (uint32_t i = threadIdx.x; i < TOKENS * TERMS * plane; i += kThreads) xs[i] = 0;  // (padding and unused tokens)
    __syncthreads();
#pragma unroll
    for (int t = 0; t < TOKENS; ++t) {
        if (t >= static_cast<int>(p.tokens)) break;
        float amax = 0.0f;
        for (uint32_t i = threadIdx.x; i < p.k; i += kThreads) amax = fmaxf(amax, finite_abs(load_x<XT>(x + static_cast<size_t>(t) * p.k, i)));
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        if (lane == 0) red[warp] = amax;
        __syncthreads();
        amax = red[0];
#pragma unroll
        for (uint32_t i = 1; i < kWarps; ++i) amax = fmaxf(amax, red[i]);
        // gain = 2^(14 - exponent(amax)): amax * gain lies in [2^14, 2^15), below the f16 maximum
        float gain = 1.0f, inv = 1.0f;
        if (amax > 0.0f) {
            int e = static_cast<int>(__float_as_uint(amax) >> 23) - 127;  // floor(log2(amax)) for normal amax
            e = max(-100, min(100, e));
            gain = __uint_as_float(static_cast<uint32_t>(127 + 14 - e) << 23);
            inv = __uint_as_float(static_cast<uint32_t>(127 - 14 + e) << 23);
        }
        if (threadIdx.x == 0) inv_gain[t] = inv;
        uint32_t* dst = xs + static_cast<size_t>(t) * TERMS * plane;
        for (uint32_t i = threadIdx.x; i < pairs; i += kThreads) {
            const float a = load_x<XT>(x + static_cast<size_t>(t) * p.k, 2 * i) * gain;
            const float b = load_x<XT>(x + static_cast<size_t>(t) * p.k, 2 * i + 1) * gain;
            const uint32_t hi = pack_f16x2(a, b);
            const uint32_t slot = x_pair_slot(2 * i);
            dst[slot] = hi;
            if (TERMS == 2) {
                // second term: what the first left, scaled up by 2^11 so that it is again a normal f16
                const float ra = (a - f16_lo_to_f32(hi)) * 2048.0f, rb = (b - f16_hi_to_f32(hi)) * 2048.0f;
                dst[plane + slot] = pack_f16x2(ra, rb);
            }
        }
        __syncthreads();
    }

    float total[TOKENS][4];
#pragma unroll
    for (int t = 0; t < TOKENS; ++t)
#pragma unroll
        for (int s = 0; s < 4; ++s) total[t][s] = 0.0f;

    const uint32_t half = lane & 1;  // which two blocks of the k-group this lane's piece covers
    auto compute = [&](uint32_t step, const uint4 (&wbuf)[4], const uint4& sbuf) {
        // the lane's 32 activations (per token and term): four 16-byte reads, lanes side by side
        uint4 xv[TOKENS][TERMS][4];
#pragma unroll
        for (int t = 0; t < TOKENS; ++t)
#pragma unroll
            for (int m = 0; m < TERMS; ++m)
#pragma unroll
                for (uint32_t j = 0; j < 4; ++j)
                    xv[t][m][j] = *reinterpret_cast<const uint4*>(xs + (static_cast<size_t>(t) * TERMS + m) * plane + ((step * 4 + j) * 32 + lane) * 4);
        const uint32_t sw[4] = {sbuf.x, sbuf.y, sbuf.z, sbuf.w};
#pragma unroll
        for (uint32_t s = 0; s < 4; ++s) {
            const uint32_t ww[4] = {wbuf[s].x, wbuf[s].y, wbuf[s].z, wbuf[s].w};
            const uint32_t sc2 = e4m3x2_to_f16x2((sw[s] >> (16 * half)) & 0xffffu);
            const float sc[2] = {f16_lo_to_f32(sc2), f16_hi_to_f32(sc2)};
#pragma unroll
            for (uint32_t blk = 0; blk < 2; ++blk) {
                float acc[TOKENS][TERMS];
#pragma unroll
                for (int t = 0; t < TOKENS; ++t)
#pragma unroll
                    for (int m = 0; m < TERMS; ++m) acc[t][m] = 0.0f;
#pragma unroll
                for (uint32_t j = 2 * blk; j < 2 * blk + 2; ++j) {
#pragma unroll
                    for (uint32_t b = 0; b < 4; ++b) {
                        const uint32_t wh = e2m1x2_to_f16x2((ww[j] >> (8 * b)) & 0xffu);
#pragma unroll
                        for (int t = 0; t < TOKENS; ++t)
#pragma unroll
                            for (int m = 0; m < TERMS; ++m) {
                                const uint32_t xw = b == 0 ? xv[t][m][j].x : b == 1 ? xv[t][m][j].y : b == 2 ? xv[t][m][j].z : xv[t][m][j].w;
                                fma2_f16(acc[t][m], wh, xw);
                            }
                    }
                }
#pragma unroll
                for (int t = 0; t < TOKENS; ++t) {
                    float a = acc[t][0];
                    if (TERMS == 2) a = fmaf(acc[t][1], 1.0f / 2048.0f, a);
                    total[t][s] = fmaf(a, sc[blk], total[t][s]);
                }
            }
        }
    };
    for (uint32_t step = 0; step < steps; step += 2) {
        if (step + 1 < steps) request(step + 1, wb, sb);
        compute(step, wa, sa);
        if (step + 1 < steps) {
            if (step + 2 < steps) request(step + 2, wa, sa);
            compute(step + 1, wb, sb);
        }
    }

    // ---- reduce over the lanes of the warp and write the warp's four rows
#pragma unroll
    for (int t = 0; t < TOKENS; ++t)
#pragma unroll
        for (int s = 0; s < 4; ++s)
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) total[t][s] += __shfl_xor_sync(0xffffffffu, total[t][s], o);
    if (lane < 4) {
#pragma unroll
        for (int t = 0; t < TOKENS; ++t) {
            if (t >= static_cast<int>(p.tokens)) break;
            const uint32_t row = row0 + 32 * lane;
            if (row >= p.n) continue;
            const float sum = lane == 0 ? total[t][0] : lane == 1 ? total[t][1] : lane == 2 ? total[t][2] : total[t][3];
            const size_t index = static_cast<size_t>(t) * p.ld_out + row;
            float y = sum * inv_gain[t] * p.alpha;
            if (p.beta != 0.0f && p.c_in)
                y = fmaf(p.beta, p.out_is_bf16 ? bf16_bits_to_float(static_cast<const uint16_t*>(p.c_in)[index])
                                               : static_cast<const float*>(p.c_in)[index], y);
            if (p.out_is_bf16) static_cast<uint16_t*>(p.out)[index] = float_to_bf16_bits(y);
            else static_cast<float*>(p.out)[index] = y;
        }
    }
}

template <typename XT, int TERMS, int TOKENS> cudaError_t launch_one(const Params& p, cudaStream_t stream) {
    auto kernel = gemv_stream_kernel<XT, TERMS, TOKENS>;
    const size_t smem = static_cast<size_t>(TOKENS) * TERMS * ((p.k / 32 + 31) / 32) * 512 * sizeof(uint32_t);
    if (smem > 200 * 1024) return cudaErrorInvalidValue;
    static size_t configured = 0;
    if (smem > 48 * 1024 && smem > configured) {
        cudaError_t st = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        if (st != cudaSuccess) return st;
        configured = smem;
    }
    const uint32_t tiles = (p.n + 127) / 128;
    kernel<<<tiles * 4, kThreads, smem, stream>>>(p);
    return cudaGetLastError();
}

// Whether the streaming kernel takes this call (one or two tokens, K a multiple of 32, 16-byte aligned operands).
inline bool supported(const Params& p) {
    return p.tokens >= 1 && p.tokens <= 2 && p.k % 32 == 0 && (reinterpret_cast<uintptr_t>(p.w) & 15) == 0 &&
           (reinterpret_cast<uintptr_t>(p.sf) & 15) == 0 && ((p.k / 2) % 16) == 0;
}

inline cudaError_t launch(const Params& p, int input_is_bf16, cudaStream_t stream) {
    if (input_is_bf16)
        return p.tokens == 1 ? launch_one<uint16_t, 1, 1>(p, stream) : launch_one<uint16_t, 1, 2>(p, stream);
    return p.tokens == 1 ? launch_one<float, 2, 1>(p, stream) : launch_one<float, 2, 2>(p, stream);
}

}  // namespace gemv_stream
}  // namespace eider
