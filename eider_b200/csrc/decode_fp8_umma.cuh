// Single-launch FP8 W8A8 decode for one to four tokens (tcgen05 kind::f8f6f4).
//
// y[t][n] = alpha * s_x[t] * s_w[n] * sum_k e4m3(xq[t][k]) * e4m3(W[n][k]),   xq[t] = e4m3(x[t] / s_x[t]),
// s_x[t] = amax(x[t]) / 448 (1 when the row is all zero): the reference's per-token dynamic activation quantizer
// (crates/eider-cuda/native/non_gemm.cu:9952-9974) folded into the GEMV.
//
// Same shape as the NVFP4 single-launch kernel: one (128-row tile, K split) item per CTA, three CTAs resident per SM;
// warp 0 streams the CTA's weight stages (128 rows x 128 bytes of K, TMA, 128-byte swizzle) and requests the first ones
// before the setup barrier; warps 2..5 find the row maxima, quantize the CTA's K slice straight into the swizzled
// operand tiles and later run the epilogue; warp 1 issues four MMAs per stage (weights on the 128 tensor-memory lanes,
// tokens on 16 columns).  K splits meet in fp32 scratch, the last CTA of a row tile sums them in split order.
// Launched as a programmatic dependent launch: everything before griddepcontrol.wait overlaps the previous kernel.
#pragma once

#include <cuda.h>

#include "common.cuh"
#include "umma.cuh"

namespace eider {
namespace decode_fp8 {

constexpr uint32_t kRows = 128;
constexpr uint32_t kCols = 16;
constexpr uint32_t kMaxTokens = 4;
constexpr uint32_t kStageK = 128;                  // bytes (= elements) of K per stage
constexpr uint32_t kWeightTile = kRows * kStageK;  // 16 KB
constexpr uint32_t kActTile = kCols * kStageK;     // 2 KB
constexpr uint32_t kMaxRing = 8;
constexpr uint32_t kMaxPer = 16;
constexpr uint32_t kThreads = 64 + 128;
constexpr uint32_t kFixedBytes = 1024 /*alignment*/ + 512 /*barriers, flags*/;
constexpr uint32_t kTmemCols = 32;

__host__ __device__ inline uint32_t smem_bytes(uint32_t per, uint32_t ring) { return kFixedBytes + ring * kWeightTile + per * kActTile; }

struct Params {
    const void* x;  // [tokens][k] bf16 or f32
    uint32_t tokens, n, k;
    uint32_t k_stages, splits, per, ring, row_tiles;
    const float* channel_scale;  // [n] or null
    void* out;                   // [tokens][ld_out]
    uint32_t ld_out;
    int out_is_bf16;
    float alpha;
    float* workspace;    // [splits][tokens][row_tiles * 128]
    uint32_t* counters;  // [row_tiles], self-resetting
    uint32_t* status;
    const float* x_scale;  // quantized-activation kernel: [tokens] scales written by the activation quantizer
    uint32_t defer_reduce; // quantized-activation kernel: leave the K splits' partial sums to splitk_reduce_kernel
};

template <typename XT> __device__ __forceinline__ void load8(const XT* p, float (&v)[8]);
template <> __device__ __forceinline__ void load8<uint16_t>(const uint16_t* p, float (&v)[8]) {
    const uint4 u = __ldg(reinterpret_cast<const uint4*>(p));
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        v[2 * j] = __uint_as_float(w[j] << 16);
        v[2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
    }
}
template <> __device__ __forceinline__ void load8<float>(const float* p, float (&v)[8]) {
    const float4 a = __ldg(reinterpret_cast<const float4*>(p)), b = __ldg(reinterpret_cast<const float4*>(p) + 1);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}

template <typename XT>
__global__ void __launch_bounds__(kThreads, 3) fp8_decode_fused_kernel(const __grid_constant__ CUtensorMap map_w, const Params p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    const uint32_t kRing = p.ring;
    uint8_t* ring_w = smem;
    uint8_t* act = ring_w + kRing * kWeightTile;  // [per][16 rows][128 B], swizzled
    uint8_t* tail = act + p.per * kActTile;
    uint64_t* full = reinterpret_cast<uint64_t*>(tail);  // [kMaxRing]
    uint64_t* empty = full + kMaxRing;                   // [kMaxRing]
    uint64_t* acc_full = empty + kMaxRing;               // [1]
    uint64_t* act_ready = acc_full + 1;                  // [1]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(act_ready + 1);
    volatile uint32_t* abort_flag = tmem_slot + 1;
    uint32_t* last_flag = tmem_slot + 2;
    float* red = reinterpret_cast<float*>(tmem_slot + 4);  // [4 warps][kMaxTokens]
    float* x_scale = red + 4 * kMaxTokens;                 // [kMaxTokens]

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t split = blockIdx.x % p.splits, rt = blockIdx.x / p.splits;
    const uint32_t stage0 = split * p.per, stage1 = min(p.k_stages, stage0 + p.per);
    const uint32_t nstages = stage1 > stage0 ? stage1 - stage0 : 0;

    if (warp >= 2) {  // operand tiles start as zeros: token rows past `tokens` and the K tail stay zero
        uint4* z = reinterpret_cast<uint4*>(act);
        for (uint32_t i = threadIdx.x - 64; i < p.per * kActTile / 16; i += 128) z[i] = make_uint4(0, 0, 0, 0);
    }
    if (threadIdx.x == 0) {
        for (uint32_t i = 0; i < kMaxRing; ++i) {
            umma::mbar_init(&full[i], 1);
            umma::mbar_init(&empty[i], 1);
        }
        umma::mbar_init(acc_full, 1);
        umma::mbar_init(act_ready, 1);
        *abort_flag = 0;
        *last_flag = 0;
        umma::fence_barrier_init();
        umma::prefetch_tensormap(&map_w);
    }
    auto load_stage = [&](uint32_t s, uint32_t slot) {
        umma::mbar_arrive_expect_tx(&full[slot], kWeightTile);
        umma::tma_load_2d(ring_w + slot * kWeightTile, &map_w, &full[slot], static_cast<int32_t>(s * kStageK), static_cast<int32_t>(rt * kRows));
    };
    // weights depend on nothing and every slot is free: the first ring is requested before the setup barrier
    const uint32_t early = min(kRing, nstages);
    if (threadIdx.x == 0)
        for (uint32_t i = 0; i < early; ++i) load_stage(stage0 + i, i);
    if (warp == 1) {
        umma::tmem_alloc(tmem_slot, kTmemCols);
        umma::tmem_relinquish();
    }
    umma::tc_fence_before();
    __syncthreads();
    umma::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    if (threadIdx.x == 0) umma::griddep_launch_dependents();

    if (warp == 0) {
        // ---------------------------------------------------------------- weight producer
        const bool leader = umma::elect_one();
        for (uint32_t it = early; it < nstages; ++it) {
            const uint32_t slot = it % kRing, phase = (it / kRing) & 1;
            if (!__all_sync(0xffffffffu, umma::mbar_wait(&empty[slot], phase ^ 1, abort_flag, p.status, umma::kTimeoutEmpty))) break;
            if (leader) load_stage(stage0 + it, slot);
            __syncwarp();
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issuer
        const bool leader = umma::elect_one();
        constexpr uint32_t idesc = umma::idesc_f8(kCols);
        const uint32_t w_lo0 = umma::desc_lo_sw128(umma::smem_u32(ring_w));
        const uint32_t a_lo0 = umma::desc_lo_sw128(umma::smem_u32(act));
        bool ok = __all_sync(0xffffffffu, umma::mbar_wait(act_ready, 0, abort_flag, p.status, umma::kTimeoutOther));
        umma::tc_fence_after();
        for (uint32_t it = 0; ok && it < nstages; ++it) {
            const uint32_t slot = it % kRing, phase = (it / kRing) & 1;
            if (!__all_sync(0xffffffffu, umma::mbar_wait(&full[slot], phase, abort_flag, p.status, umma::kTimeoutFull))) { ok = false; break; }
            umma::tc_fence_after();
            if (leader) {
                const uint32_t w_lo = w_lo0 + slot * (kWeightTile >> 4), a_lo = a_lo0 + it * (kActTile >> 4);
#pragma unroll
                for (uint32_t j = 0; j < 4; ++j)  // K past the end is zero on both sides (TMA fill, cleared tiles)
                    umma::mma_f8(tmem_base, umma::make_desc(w_lo + j * 2, umma::kDescHiSw128), umma::make_desc(a_lo + j * 2, umma::kDescHiSw128),
                                 idesc, (it > 0 || j > 0) ? 1u : 0u);
                umma::tc_commit(&empty[slot]);
            }
            __syncwarp();
        }
        if (ok && leader) umma::tc_commit(acc_full);
        __syncwarp();
    } else {
        // ---------------------------------------------------------------- quantize the slice, then epilogue
        const uint32_t te = threadIdx.x - 64;  // 0..127
        const uint32_t quad = warp & 3;
        umma::griddep_wait();  // x may be the previous kernel's output; scratch, counters and the output are shared with it
        const XT* x = static_cast<const XT*>(p.x);
        // row maxima over the whole K (the scale is per token, not per slice)
        float amax[kMaxTokens];
#pragma unroll
        for (uint32_t m = 0; m < kMaxTokens; ++m) amax[m] = 0.0f;
        for (uint32_t h = te; h < p.k / 8; h += 128) {
#pragma unroll
            for (uint32_t m = 0; m < kMaxTokens; ++m) {
                if (m >= p.tokens) break;
                float v[8];
                load8<XT>(x + static_cast<size_t>(m) * p.k + h * 8, v);
#pragma unroll
                for (int i = 0; i < 8; ++i) amax[m] = fmaxf(amax[m], finite_abs(v[i]));
            }
        }
#pragma unroll
        for (uint32_t m = 0; m < kMaxTokens; ++m) {
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) amax[m] = fmaxf(amax[m], __shfl_xor_sync(0xffffffffu, amax[m], o));
            if (lane == 0) red[quad * kMaxTokens + m] = amax[m];
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        float s[kMaxTokens];
#pragma unroll
        for (uint32_t m = 0; m < kMaxTokens; ++m) {
            const float a = fmaxf(fmaxf(red[m], red[kMaxTokens + m]), fmaxf(red[2 * kMaxTokens + m], red[3 * kMaxTokens + m]));
            s[m] = a == 0.0f ? 1.0f : __fdiv_rn(a, 448.0f);
            if (te == m) x_scale[m] = s[m];
        }
        // the CTA's K slice -> e4m3 codes in the swizzled operand tiles (8 elements = 8 bytes per thread and pass)
        const uint32_t k_begin = stage0 * kStageK, k_end = min(p.k, stage1 * kStageK);
        for (uint32_t e0 = k_begin + te * 8; e0 < k_end; e0 += 128 * 8) {
            const uint32_t ls = (e0 - k_begin) / kStageK, e = (e0 - k_begin) % kStageK;
#pragma unroll
            for (uint32_t m = 0; m < kMaxTokens; ++m) {
                if (m >= p.tokens) break;
                float v[8];
                load8<XT>(x + static_cast<size_t>(m) * p.k + e0, v);
                uint32_t w[2] = {0, 0};
#pragma unroll
                for (int i = 0; i < 8; ++i) w[i >> 2] |= static_cast<uint32_t>(e4m3_satfinite(__fdiv_rn(v[i], s[m]))) << (8 * (i & 3));
                uint8_t* dst = act + ls * kActTile + m * 128 + (((e >> 4) ^ (m & 7)) << 4) + (e & 15);
                *reinterpret_cast<uint2*>(dst) = make_uint2(w[0], w[1]);
            }
        }
        umma::fence_proxy_async();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (te == 0) umma::mbar_arrive(act_ready);

        bool ok = umma::mbar_wait(acc_full, 0, abort_flag, p.status, umma::kTimeoutTmemFull);
        if (ok) {
            umma::tc_fence_after();
            uint32_t raw[16];
            if (nstages > 0) {
                umma::tmem_load_32x16(tmem_base + ((quad * 32) << 16), raw);
                umma::tmem_load_wait();
            } else {
#pragma unroll
                for (int i = 0; i < 16; ++i) raw[i] = 0;
            }
            const uint32_t row = rt * kRows + quad * 32 + lane;
            const bool row_ok = row < p.n;
            const uint32_t padded_rows = p.row_tiles * kRows;
            const float rs = p.alpha * ((p.channel_scale && row_ok) ? p.channel_scale[row] : 1.0f);
            auto emit = [&](uint32_t m, float sum) {
                const size_t index = static_cast<size_t>(m) * p.ld_out + row;
                const float v = sum * x_scale[m] * rs;
                if (p.out_is_bf16) static_cast<uint16_t*>(p.out)[index] = float_to_bf16_bits(v);
                else static_cast<float*>(p.out)[index] = v;
            };
            if (p.splits == 1) {
                if (row_ok)
#pragma unroll
                    for (uint32_t m = 0; m < kMaxTokens; ++m)
                        if (m < p.tokens) emit(m, __uint_as_float(raw[m]));
            } else {
#pragma unroll
                for (uint32_t m = 0; m < kMaxTokens; ++m)
                    if (m < p.tokens) p.workspace[(static_cast<size_t>(split) * p.tokens + m) * padded_rows + row] = __uint_as_float(raw[m]);
                __threadfence();
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (te == 0) {
                    const uint32_t prev = atomicAdd(&p.counters[rt], 1u);
                    *last_flag = (prev == p.splits - 1) ? 1u : 0u;
                    if (prev == p.splits - 1) p.counters[rt] = 0;
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (*last_flag) {
                    __threadfence();
                    if (row_ok) {
                        // the partials of every token and of eight splits at a time are requested before any is used (one
                        // memory round trip per eight splits, not per token); each token is summed in split order
                        float sum[kMaxTokens];
#pragma unroll
                        for (uint32_t m = 0; m < kMaxTokens; ++m) sum[m] = 0.0f;
                        for (uint32_t s0 = 0; s0 < p.splits; s0 += 8) {
                            float part[kMaxTokens][8];
#pragma unroll
                            for (uint32_t m = 0; m < kMaxTokens; ++m)
#pragma unroll
                                for (uint32_t u = 0; u < 8; ++u)
                                    part[m][u] = (m < p.tokens && s0 + u < p.splits)
                                                     ? __ldcg(&p.workspace[(static_cast<size_t>(s0 + u) * p.tokens + m) * padded_rows + row])
                                                     : 0.0f;
#pragma unroll
                            for (uint32_t m = 0; m < kMaxTokens; ++m)
#pragma unroll
                                for (uint32_t u = 0; u < 8; ++u) sum[m] += part[m][u];
                        }
#pragma unroll
                        for (uint32_t m = 0; m < kMaxTokens; ++m)
                            if (m < p.tokens) emit(m, sum[m]);
                    }
                }
            }
        }
    }
    umma::tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        umma::tc_fence_after();
        umma::tmem_dealloc(tmem_base, kTmemCols);
    }
}

// ---- activations already quantized (1..64 tokens) ---------------------------------------------------------------------
// The per-token quantizer has run as its own kernel (the producer of x, or the reference's batch quantizer); this kernel is
// the same one-item-per-CTA GEMV with nothing to compute before the MMAs: every ring slot holds a weight stage and the
// matching stage of the activation codes (a tiled TMA load of COLS rows x 128 bytes, rows past `tokens` arrive as zeros),
// the activation half being requested only once the kernel before this one has finished.
__host__ __device__ inline uint32_t quantized_smem_bytes(uint32_t ring, uint32_t cols) { return kFixedBytes + ring * (kWeightTile + cols * kStageK); }

template <int COLS>
__global__ void __launch_bounds__(kThreads, 3) fp8_decode_quantized_kernel(const __grid_constant__ CUtensorMap map_w,
                                                                          const __grid_constant__ CUtensorMap map_x, const Params p) {
    constexpr uint32_t kAct = COLS * kStageK;
    constexpr uint32_t kTmem = COLS < 32 ? 32 : COLS;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    const uint32_t kRing = p.ring;
    uint8_t* ring_w = smem;
    uint8_t* ring_a = ring_w + kRing * kWeightTile;  // [ring][COLS rows][128 B], swizzled
    uint8_t* tail = ring_a + kRing * kAct;
    uint64_t* full = reinterpret_cast<uint64_t*>(tail);  // [kMaxRing]: two arrivals, the weight half and the activation half
    uint64_t* empty = full + kMaxRing;                   // [kMaxRing]
    uint64_t* acc_full = empty + kMaxRing;               // [1]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 2);
    volatile uint32_t* abort_flag = tmem_slot + 1;
    uint32_t* last_flag = tmem_slot + 2;

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t split = blockIdx.x % p.splits, rt = blockIdx.x / p.splits;
    const uint32_t stage0 = split * p.per, stage1 = min(p.k_stages, stage0 + p.per);
    const uint32_t nstages = stage1 > stage0 ? stage1 - stage0 : 0;

    if (threadIdx.x == 0) {
        for (uint32_t i = 0; i < kMaxRing; ++i) {
            umma::mbar_init(&full[i], 2);
            umma::mbar_init(&empty[i], 1);
        }
        umma::mbar_init(acc_full, 1);
        *abort_flag = 0;
        *last_flag = 0;
        umma::fence_barrier_init();
        umma::prefetch_tensormap(&map_w);
        umma::prefetch_tensormap(&map_x);
    }
    auto load_weights = [&](uint32_t s, uint32_t slot) {
        umma::mbar_arrive_expect_tx(&full[slot], kWeightTile);
        umma::tma_load_2d(ring_w + slot * kWeightTile, &map_w, &full[slot], static_cast<int32_t>(s * kStageK), static_cast<int32_t>(rt * kRows));
    };
    auto load_activation = [&](uint32_t s, uint32_t slot) {
        umma::mbar_arrive_expect_tx(&full[slot], kAct);
        umma::tma_load_2d(ring_a + slot * kAct, &map_x, &full[slot], static_cast<int32_t>(s * kStageK), 0);
    };
    // weights depend on nothing and every slot is free: the first ring is requested before the setup barrier
    const uint32_t early = min(kRing, nstages);
    if (threadIdx.x == 0)
        for (uint32_t i = 0; i < early; ++i) load_weights(stage0 + i, i);
    if (warp == 1) {
        umma::tmem_alloc(tmem_slot, kTmem);
        umma::tmem_relinquish();
    }
    umma::tc_fence_before();
    __syncthreads();
    umma::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    if (threadIdx.x == 0) umma::griddep_launch_dependents();

    if (warp == 0) {
        // ---------------------------------------------------------------- producer
        const bool leader = umma::elect_one();
        umma::griddep_wait();  // the activation codes are the output of the kernel before this one
        if (leader)
            for (uint32_t i = 0; i < early; ++i) load_activation(stage0 + i, i);
        __syncwarp();
        for (uint32_t it = early; it < nstages; ++it) {
            const uint32_t slot = it % kRing, phase = (it / kRing) & 1;
            if (!__all_sync(0xffffffffu, umma::mbar_wait(&empty[slot], phase ^ 1, abort_flag, p.status, umma::kTimeoutEmpty))) break;
            if (leader) {
                load_weights(stage0 + it, slot);
                load_activation(stage0 + it, slot);
            }
            __syncwarp();
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issuer
        const bool leader = umma::elect_one();
        constexpr uint32_t idesc = umma::idesc_f8(COLS);
        const uint32_t w_lo0 = umma::desc_lo_sw128(umma::smem_u32(ring_w));
        const uint32_t a_lo0 = umma::desc_lo_sw128(umma::smem_u32(ring_a));
        bool ok = true;
        for (uint32_t it = 0; ok && it < nstages; ++it) {
            const uint32_t slot = it % kRing, phase = (it / kRing) & 1;
            if (!__all_sync(0xffffffffu, umma::mbar_wait(&full[slot], phase, abort_flag, p.status, umma::kTimeoutFull))) { ok = false; break; }
            umma::tc_fence_after();
            if (leader) {
                const uint32_t w_lo = w_lo0 + slot * (kWeightTile >> 4), a_lo = a_lo0 + slot * (kAct >> 4);
#pragma unroll
                for (uint32_t j = 0; j < 4; ++j)  // K past the end is zero on both sides (TMA fill)
                    umma::mma_f8(tmem_base, umma::make_desc(w_lo + j * 2, umma::kDescHiSw128), umma::make_desc(a_lo + j * 2, umma::kDescHiSw128),
                                 idesc, (it > 0 || j > 0) ? 1u : 0u);
                umma::tc_commit(&empty[slot]);
            }
            __syncwarp();
        }
        if (ok && leader) umma::tc_commit(acc_full);
        __syncwarp();
    } else {
        // ---------------------------------------------------------------- epilogue
        const uint32_t te = threadIdx.x - 64;  // 0..127
        const uint32_t quad = warp & 3;
        umma::griddep_wait();  // scratch, counters and the output are shared with the kernel before this one
        bool ok = umma::mbar_wait(acc_full, 0, abort_flag, p.status, umma::kTimeoutTmemFull);
        if (ok) {
            umma::tc_fence_after();
            const uint32_t row = rt * kRows + quad * 32 + lane;
            const bool row_ok = row < p.n;
            const uint32_t padded_rows = p.row_tiles * kRows;
            const float rs = p.alpha * ((p.channel_scale && row_ok) ? p.channel_scale[row] : 1.0f);
            auto emit = [&](uint32_t m, float sum) {
                const size_t index = static_cast<size_t>(m) * p.ld_out + row;
                const float v = sum * __ldg(p.x_scale + m) * rs;
                if (p.out_is_bf16) static_cast<uint16_t*>(p.out)[index] = float_to_bf16_bits(v);
                else static_cast<float*>(p.out)[index] = v;
            };
            // sixteen tokens at a time: accumulator columns -> output, or -> this split's partial sums
#pragma unroll 1
            for (uint32_t m0 = 0; m0 < p.tokens; m0 += 16) {
                uint32_t raw[16];
                if (nstages > 0) {
                    umma::tmem_load_32x16(tmem_base + ((quad * 32) << 16) + m0, raw);
                    umma::tmem_load_wait();
                } else {
#pragma unroll
                    for (int i = 0; i < 16; ++i) raw[i] = 0;
                }
#pragma unroll
                for (uint32_t i = 0; i < 16; ++i) {
                    const uint32_t m = m0 + i;
                    if (m >= p.tokens) break;
                    if (p.splits == 1) {
                        if (row_ok) emit(m, __uint_as_float(raw[i]));
                    } else {
                        p.workspace[(static_cast<size_t>(split) * p.tokens + m) * padded_rows + row] = __uint_as_float(raw[i]);
                    }
                }
            }
            if (p.splits > 1 && !p.defer_reduce) {
                __threadfence();
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (te == 0) {
                    const uint32_t prev = atomicAdd(&p.counters[rt], 1u);
                    *last_flag = (prev == p.splits - 1) ? 1u : 0u;
                    if (prev == p.splits - 1) p.counters[rt] = 0;
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (*last_flag) {
                    __threadfence();
                    if (row_ok) {
                        // eight tokens x four splits are requested before any is used; each token is summed in split order
#pragma unroll 1
                        for (uint32_t m0 = 0; m0 < p.tokens; m0 += 8) {
                            float sum[8];
#pragma unroll
                            for (uint32_t i = 0; i < 8; ++i) sum[i] = 0.0f;
                            for (uint32_t s0 = 0; s0 < p.splits; s0 += 4) {
                                float part[8][4];
#pragma unroll
                                for (uint32_t i = 0; i < 8; ++i)
#pragma unroll
                                    for (uint32_t u = 0; u < 4; ++u)
                                        part[i][u] = (m0 + i < p.tokens && s0 + u < p.splits)
                                                         ? __ldcg(&p.workspace[(static_cast<size_t>(s0 + u) * p.tokens + m0 + i) * padded_rows + row])
                                                         : 0.0f;
#pragma unroll
                                for (uint32_t i = 0; i < 8; ++i)
#pragma unroll
                                    for (uint32_t u = 0; u < 4; ++u) sum[i] += part[i][u];
                            }
#pragma unroll
                            for (uint32_t i = 0; i < 8; ++i)
                                if (m0 + i < p.tokens) emit(m0 + i, sum[i]);
                        }
                    }
                }
            }
        }
    }
    umma::tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        umma::tc_fence_after();
        umma::tmem_dealloc(tmem_base, kTmem);
    }
}

// Sums the K splits' partial sums of fp8_decode_quantized_kernel when many tokens share the launch: the one CTA per row tile
// that arrives last would need a memory round trip per eight tokens, this kernel spreads the same sums (in split order) over
// the whole device.  One thread per (token, output row); launched as a programmatic dependent launch.
__global__ void __launch_bounds__(256) splitk_reduce_kernel(const Params p) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const uint32_t row = blockIdx.x * 256 + threadIdx.x, m = blockIdx.y;
    if (row >= p.n) return;
    const uint32_t padded_rows = p.row_tiles * kRows;
    float sum = 0.0f;
    for (uint32_t s0 = 0; s0 < p.splits; s0 += 8) {
        float part[8];
#pragma unroll
        for (uint32_t u = 0; u < 8; ++u)
            part[u] = s0 + u < p.splits ? __ldcg(&p.workspace[(static_cast<size_t>(s0 + u) * p.tokens + m) * padded_rows + row]) : 0.0f;
#pragma unroll
        for (uint32_t u = 0; u < 8; ++u) sum += part[u];
    }
    const float v = sum * __ldg(p.x_scale + m) * p.alpha * (p.channel_scale ? p.channel_scale[row] : 1.0f);
    const size_t index = static_cast<size_t>(m) * p.ld_out + row;
    if (p.out_is_bf16) static_cast<uint16_t*>(p.out)[index] = float_to_bf16_bits(v);
    else static_cast<float*>(p.out)[index] = v;
}

}  // namespace decode_fp8
}  // namespace eider
