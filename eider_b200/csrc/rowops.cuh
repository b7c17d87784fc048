// Row reductions and activation formulas shared by the fused producers of the NVFP4 quantizer and by the staged
// kernels the same operators are split into (norm / activation to f32, then the plain quantizer).  The fused and the
// staged path must produce the same bytes (the reference's own criterion,
// crates/eider-cuda/src/kernels/non_gemm.rs:19687-19750), so both take every sum and every product from here: one
// order of additions, explicit roundings, no contraction left to the compiler.
#pragma once

#include "common.cuh"

namespace eider {
namespace rowops {

// Per-thread part of a row's sum of squares: float4 loads strided by the CTA, FMAs in element order.
__device__ __forceinline__ float thread_sum_squares_f4(const float* __restrict__ x, uint32_t cols) {
    float ss = 0.0f;
    for (uint32_t i = threadIdx.x; i < cols / 4; i += blockDim.x) {
        const float4 v = __ldg(reinterpret_cast<const float4*>(x) + i);
        ss = fmaf(v.x, v.x, ss);
        ss = fmaf(v.y, v.y, ss);
        ss = fmaf(v.z, v.z, ss);
        ss = fmaf(v.w, v.w, ss);
    }
    return ss;
}

// The same for rows that cannot be read as float4 (any length, any alignment).
__device__ __forceinline__ float thread_sum_squares_scalar(const float* __restrict__ x, uint32_t cols) {
    float ss = 0.0f;
    for (uint32_t i = threadIdx.x; i < cols; i += blockDim.x) {
        const float v = __ldg(x + i);
        ss = fmaf(v, v, ss);
    }
    return ss;
}

// CTA-wide sum in a fixed order: butterfly inside each warp, then the warp sums added in warp order by every thread.
// `red` holds one float per warp (at most 32); the two barriers make it reusable right away.
__device__ __forceinline__ float block_sum_ordered(float v, float* red) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float total = 0.0f;
    for (uint32_t w = 0; w < (blockDim.x >> 5); ++w) total += red[w];
    __syncthreads();
    return total;
}

// 1 / sqrt(mean + eps) with the reference's operations (crates/eider-cuda/native/non_gemm.cu:663).
__device__ __forceinline__ float inverse_rms(float sum_squares, uint32_t cols, float eps) {
    return rsqrtf(__fadd_rn(__fdiv_rn(sum_squares, static_cast<float>(cols)), eps));
}

// x * inverse_rms * weight, left to right (non_gemm.cu:665).
__device__ __forceinline__ float normed(float x, float inv, float w) { return __fmul_rn(__fmul_rn(x, inv), w); }

// x * inverse_rms * weight + residual: the product chain, then one fused multiply-add (non_gemm.cu:724-725 as nvcc
// contracts it).
__device__ __forceinline__ float normed_add(float x, float inv, float w, float r) { return fmaf(__fmul_rn(x, inv), w, r); }

// gate * sigmoid(gate) * up with sigmoid = 1 / (1 + expf(-gate)) (non_gemm.cu:576-577).
__device__ __forceinline__ float silu_sigmoid_mul(float g, float u) {
    const float sigmoid = __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-g)));
    return __fmul_rn(__fmul_rn(g, sigmoid), u);
}

// (gate / (1 + expf(-gate))) * up: the spelling of the staged and routed kernels (non_gemm.cu:1369, 2837-2840).
__device__ __forceinline__ float silu_div_mul(float g, float u) { return __fmul_rn(__fdiv_rn(g, __fadd_rn(1.0f, expf(-g))), u); }

// tanh-approximated GELU(gate) * up (non_gemm.cu:446-451).
__device__ __forceinline__ float gelu_tanh_mul(float g, float u) {
    const float cubic = __fmul_rn(__fmul_rn(g, g), g);
    const float inner = __fmul_rn(0.7978845608028654f, fmaf(0.044715f, cubic, g));
    const float gelu = __fmul_rn(__fmul_rn(0.5f, g), __fadd_rn(1.0f, tanhf(inner)));
    return __fmul_rn(gelu, u);
}

}  // namespace rowops
}  // namespace eider
