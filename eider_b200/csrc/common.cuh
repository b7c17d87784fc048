// Shared device/host helpers for the quantized-linear kernels: NVFP4 / FP8 codecs and the
// 128x4 tiled scale layout.  Numeric semantics follow the reference's host code
// (crates/eider-cuda/src/format.rs) and are checked bit-for-bit against the CPU oracle.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp4.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>

namespace eider {

constexpr float kE2M1Max = 6.0f;
constexpr float kRowScaleDivisor = 2688.0f;  // 6 * 448: e2m1 max times e4m3 max

__host__ __device__ inline uint32_t round_up_u32(uint32_t v, uint32_t m) { return (v + m - 1) / m * m; }

// Bytes of the tiled UE4M3 scale buffer for `outer` rows of `inner` elements
// (crates/eider-cuda/src/format.rs:194-198).
__host__ __device__ inline size_t scale_layout_len(size_t outer, size_t inner) {
    size_t blocks = (inner + 15) / 16;
    size_t padded = (blocks + 3) / 4 * 4;
    return (outer + 127) / 128 * 128 * padded;
}

// Byte offset of (row `outer`, 16-block `kb`) in the 128-row x 4-block tile order
// (crates/eider-cuda/src/format.rs:208-218).  One 512-byte tile holds 128 rows x 4 blocks as
// [row % 32][row / 32 % 4][kb % 4], which is also the shape one tcgen05.cp 32x128b copy wants.
__host__ __device__ inline size_t tiled_scale_offset(uint32_t outer, uint32_t kb, uint32_t inner) {
    uint32_t blocks = (inner + 15) / 16;
    uint32_t padded = round_up_u32(blocks, 4);
    uint32_t in_tile = outer % 128;
    size_t base = (static_cast<size_t>(kb / 4) * 4 + static_cast<size_t>(outer / 128) * padded) * 128;
    return base + (in_tile % 32) * 16 + (in_tile / 32) * 4 + (kb % 4);
}

// E4M3 byte -> f32 (crates/eider-cuda/src/format.rs:121-133).
__host__ __device__ inline float e4m3_value(uint8_t code) {
    uint32_t sign = static_cast<uint32_t>(code & 0x80) << 24;
    uint32_t exp = (code >> 3) & 0x0f;
    uint32_t mant = code & 0x07;
    uint32_t bits;
    if (exp == 0) {
        float v = static_cast<float>(mant) * 0.001953125f;  // 2^-9
#ifdef __CUDA_ARCH__
        bits = __float_as_uint(v) | sign;
        return __uint_as_float(bits);
#else
        return sign ? -v : v;
#endif
    }
    if (exp == 0x0f && mant == 0x07) bits = sign | 0x7fffffffu;
    else bits = sign | ((exp + 120u) << 23) | (mant << 20);
#ifdef __CUDA_ARCH__
    return __uint_as_float(bits);
#else
    float f;
    memcpy(&f, &bits, 4);
    return f;
#endif
}

// Residual NVFP4 expansion of activation rows (defined beside its kernel): scale bytes go to the 128 x 4 tiled layout of a GEMM
// operand when operand_cols is 0, else to [64-element block][operand_cols rows][16 bytes].
cudaError_t expand_nvfp4_terms_launch(const void* input, int input_is_bf16, uint8_t* packed, uint8_t* scales, float* col_scale,
                                      uint32_t tokens, uint32_t in_features, uint32_t terms, uint32_t operand_cols, cudaStream_t stream);

#ifdef __CUDACC__

// E2M1 nibble -> f32 (crates/eider-cuda/src/format.rs:78-96).
__device__ __forceinline__ float e2m1_value(uint32_t nibble) {
    uint32_t mag = nibble & 7u;
    uint32_t e = mag >> 1, m = mag & 1u;
    uint32_t bits = e == 0 ? m * 0x3f000000u : (((e + 126u) << 23) | (m << 22));
    return __uint_as_float(bits | ((nibble & 8u) << 28));
}

// Positive finite f32 -> UE4M3 byte, nearest-even, saturating at 448
// (crates/eider-cuda/src/format.rs:151-167 == __nv_cvt_float_to_fp8(SATFINITE, E4M3)).
__device__ __forceinline__ uint8_t ue4m3_code(float v) {
    return static_cast<uint8_t>(__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3));
}

// Signed E4M3, saturating, NaN -> 0x7f: the conversion the reference's FP8 quantizers use
// (crates/eider-cuda/native/non_gemm.cu:9971-9972).
__device__ __forceinline__ uint8_t e4m3_satfinite(float v) {
    return static_cast<uint8_t>(__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3));
}

// Two f32 -> one byte of E2M1 codes, `lo` in the low nibble (format.rs:44-110).
__device__ __forceinline__ uint8_t e2m1x2_code(float lo, float hi) {
    return static_cast<uint8_t>(__nv_cvt_float2_to_fp4x2(make_float2(lo, hi), __NV_E2M1, cudaRoundNearest));
}

__device__ __forceinline__ float bf16_bits_to_float(uint16_t b) { return __uint_as_float(static_cast<uint32_t>(b) << 16); }

// f32 -> bf16 bits, nearest-even (crates/eider-cuda/src/format.rs:368-376).
__device__ __forceinline__ uint16_t float_to_bf16_bits(float v) {
    return __bfloat16_as_ushort(__float2bfloat16_rn(v));
}

// Correctly rounded division by a divisor that is reused many times.  With r = RN(1/d) correctly rounded,
// q0 = RN(x r), e = x - q0 d (exact in one FMA) and q = RN(q0 + e r) is the correctly rounded x / d (Markstein)
// whenever nothing under- or overflows on the way.  The quantizers only depend on quotients of ordinary
// magnitude: a quotient that underflows is far below every E2M1 / E4M3 rounding boundary and encodes to the same
// code either way, zeros keep their sign through q0, and an overflowing q0 is passed through as the infinity the
// IEEE division would give.  Divisors outside 2^-20 .. 2^20 (where e itself could underflow) use __fdiv_rn.
struct Divisor {
    float d, r;
    bool fast;
};
__device__ __forceinline__ Divisor make_divisor(float d) {
    Divisor D;
    D.d = d;
    D.r = __frcp_rn(d);
    D.fast = d > 9.5367431640625e-07f && d < 1048576.0f;
    return D;
}
__device__ __forceinline__ float div_rn(float x, const Divisor& D) {
    if (!D.fast) return __fdiv_rn(x, D.d);
    const float q0 = x * D.r;
    const float e = fmaf(-q0, D.d, x);
    const float q = fmaf(e, D.r, q0);
    const float aq = fabsf(q0);
    return (aq == 0.0f || aq == __int_as_float(0x7f800000)) ? q0 : q;
}
// The same quotient for a finite x and a divisor in the fast range, without the two comparisons: x * r never overflows for
// the quantizers' operands, an underflowed q0 = +-0 leaves q = RN(x r) = q0, and the only case where q and q0 differ in
// more than the last place's correction is x = -0 (e = +0, q = +0), which the sign of x restores.  NaN stays NaN.
__device__ __forceinline__ float div_rn_finite(float x, const Divisor& D) {
    const float q0 = x * D.r;
    const float e = fmaf(-q0, D.d, x);
    return copysignf(fmaf(e, D.r, q0), x);
}
// Row scale of the on-the-fly quantizer: the smallest power of two g with amax / g <= 2688 (1 for amax == 0), so that
// x / g is exact and the largest block scale still fits E4M3.  2688 = 1.3125 * 2^11.
__device__ __forceinline__ float row_scale_pow2(float amax) {
    if (!(amax > 0.0f)) return 1.0f;
    const uint32_t bits = __float_as_uint(amax);
    int ge = static_cast<int>(bits >> 23) - 11 + ((bits & 0x7fffffu) > 0x280000u ? 1 : 0);
    ge = max(1, min(254, ge));
    return __uint_as_float(static_cast<uint32_t>(ge) << 23);
}
// 1 / g for a power of two g in the normal range (exact).
__device__ __forceinline__ float pow2_reciprocal(float g) { return __uint_as_float((254u << 23) - __float_as_uint(g)); }

// |v| for finite v, 0 otherwise (NaN compares false): the quantizers ignore non-finite values in maxima.
__device__ __forceinline__ float finite_abs(float v) {
    const float a = fabsf(v);
    return a < __int_as_float(0x7f800000) ? a : 0.0f;
}
// amax / 6 correctly rounded (6 is far from every hazard of the scheme above).
__device__ __forceinline__ float div6_rn(float a) {
    const float r = 0.16666667163372039794921875f;  // RN(1/6)
    const float q0 = a * r;
    const float e = fmaf(-q0, 6.0f, a);
    const float q = fmaf(e, r, q0);
    return (q0 > 1e-30f && q0 < 1e30f) ? q : __fdiv_rn(a, 6.0f);
}

// SiLU(gate) * up of the routed-MoE kernels: (g / (1 + e^-g)) * u (crates/eider-cuda/native/non_gemm.cu:2837-2840) with the
// hardware exponential and reciprocal, which is also what the reference's build (--use_fast_math) turns that line into.
// The stand-alone quantizer and the grouped GEMM's fused epilogue both call this, so their bytes agree; against a host
// libm the last place of the exponential may differ.
__device__ __forceinline__ float moe_silu_mul(float g, float u) { return __fmul_rn(__fdividef(g, __fadd_rn(1.0f, __expf(-g))), u); }

// Quantize one 16-element block already divided by the input scale.  Returns the scale byte and
// writes 8 packed bytes.  Order of operations: crates/eider-cuda/native/non_gemm.cu:120-153.
__device__ __forceinline__ uint8_t quantize_block16(const float (&v)[16], uint32_t valid, uint2* packed_out) {
    if (valid == 16) {
        // Whole blocks without an infinity: one max per element (fmaxf drops NaNs as the maximum below does, an infinity
        // shows in the result) and the quotient without its special-case comparisons.  Same bytes as the path below.
        float m = 0.0f;
#pragma unroll
        for (int i = 0; i < 16; ++i) m = fmaxf(m, fabsf(v[i]));
        if (m != __int_as_float(0x7f800000)) {
            const uint8_t sc = m == 0.0f ? 0 : ue4m3_code(div6_rn(m));
            const float s = e4m3_value(sc);
            uint32_t w[2] = {0u, 0u};
            if (s != 0.0f) {
                const Divisor ds = make_divisor(s);  // (an E4M3 value: always inside the fast range)
#pragma unroll
                for (int i = 0; i < 16; i += 2)
                    w[i / 8] |= static_cast<uint32_t>(e2m1x2_code(div_rn_finite(v[i], ds), div_rn_finite(v[i + 1], ds))) << ((i % 8) * 4);
            }
            *packed_out = make_uint2(w[0], w[1]);
            return sc;
        }
    }
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 16; ++i)
        if (static_cast<uint32_t>(i) < valid) amax = fmaxf(amax, finite_abs(v[i]));
    uint8_t sc = amax == 0.0f ? 0 : ue4m3_code(div6_rn(amax));
    float s = e4m3_value(sc);
    const Divisor ds = make_divisor(s == 0.0f ? 1.0f : s);
    uint32_t w[2] = {0u, 0u};
#pragma unroll
    for (int i = 0; i < 16; i += 2) {
        float lo = (s == 0.0f || static_cast<uint32_t>(i) >= valid) ? 0.0f : div_rn(v[i], ds);
        float hi = (s == 0.0f || static_cast<uint32_t>(i + 1) >= valid) ? 0.0f : div_rn(v[i + 1], ds);
        uint32_t byte = e2m1x2_code(lo, hi);
        if (static_cast<uint32_t>(i + 1) >= valid) byte &= 0x0fu;
        if (static_cast<uint32_t>(i) >= valid) byte = 0;
        w[i / 8] |= byte << ((i % 8) * 4);
    }
    *packed_out = make_uint2(w[0], w[1]);
    return sc;
}

#endif  // __CUDACC__

}  // namespace eider
