// Single-launch NVFP4 W4A16 decode GEMV for one or two tokens (tcgen05).
//
// The weight matrix is the only thing that moves: 128 output features x 128 bytes of K per stage stream through a
// deep TMA ring straight into the tensor cores.  The activation never goes through global memory in quantized form:
// each CTA owns one K split (fixed for the whole launch), and its four epilogue warps expand that slice of x into
// residual NVFP4 terms (x ~= sum_j g_j deq(q_j), g_j = g_0 / 4^j, g_0 from the slice maximum) directly into
// shared-memory operand tiles in the 128-byte-swizzled K-major layout the MMA descriptors expect, while the producer
// warp is already prefetching weights.  Partial sums of the K splits meet in a small fp32 scratch; the last CTA of a
// row tile reduces them in split order.
#pragma once

#include <cuda.h>

#include "common.cuh"
#include "umma.cuh"

namespace eider {
namespace decode {

constexpr uint32_t kRows = 128;          // output features per tile (MMA M)
constexpr uint32_t kCols = 16;           // MMA N: tokens x terms, zero padded
constexpr uint32_t kStageK = 128;        // bytes of K per stage
constexpr uint32_t kMaxLocalStages = 8;  // stages of one K split (its activation slice stays resident)
constexpr uint32_t kRing = 10;           // weight stages in flight
constexpr uint32_t kThreads = 192;
constexpr uint32_t kWeightTile = kRows * kStageK;  // 16 KB
constexpr uint32_t kSfTile = 4 * 512;              // scales of one stage for 128 rows
constexpr uint32_t kActTile = kCols * kStageK;     // 2 KB
constexpr uint32_t kSmemBytes = kRing * (kWeightTile + kSfTile) + kMaxLocalStages * (kActTile + kSfTile) + 1024 + 512;
constexpr uint32_t kTmemCols = 64;       // 2 x 16 accumulator columns + 16 + 16 scale columns

struct Params {
    const void* x;            // [tokens][k] bf16 or f32
    uint32_t tokens, n, k;
    uint32_t k_stages;        // ceil(k / 256)
    uint32_t splits, per;     // K splits and stages per split (per <= kMaxLocalStages)
    uint32_t row_tiles;
    const uint8_t* sf_w;      // tiled weight scales
    uint32_t sf_tile_stride;
    void* out;
    const void* c_in;
    uint32_t ld_out;
    int out_is_bf16;
    float alpha, beta;
    float* workspace;         // [splits][tokens][row_tiles * 128]
    uint32_t* counters;       // [row_tiles], self-resetting
    uint32_t* status;
};

template <typename XT> __device__ __forceinline__ void load16(const XT* p, float (&v)[16]);
template <> __device__ __forceinline__ void load16<uint16_t>(const uint16_t* p, float (&v)[16]) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const uint4 u = __ldg(reinterpret_cast<const uint4*>(p) + h);
        const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            v[8 * h + 2 * j] = __uint_as_float(w[j] << 16);
            v[8 * h + 2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
        }
    }
}
template <> __device__ __forceinline__ void load16<float>(const float* p, float (&v)[16]) {
#pragma unroll
    for (int h = 0; h < 4; ++h) {
        const float4 f = __ldg(reinterpret_cast<const float4*>(p) + h);
        v[4 * h] = f.x; v[4 * h + 1] = f.y; v[4 * h + 2] = f.z; v[4 * h + 3] = f.w;
    }
}

template <int TERMS, typename XT>
__global__ void __launch_bounds__(kThreads, 1) nvfp4_decode_fused_kernel(const __grid_constant__ CUtensorMap map_w, const Params p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    uint8_t* ring_w = smem;
    uint8_t* act = ring_w + kRing * kWeightTile;            // [kMaxLocalStages][16 rows][128 B], swizzled
    uint8_t* ring_sf = act + kMaxLocalStages * kActTile;    // [kRing][2 KB]
    uint8_t* act_sf = ring_sf + kRing * kSfTile;            // [kMaxLocalStages][2 KB]
    uint8_t* tail = act_sf + kMaxLocalStages * kSfTile;
    uint64_t* full = reinterpret_cast<uint64_t*>(tail);     // [kRing]
    uint64_t* empty = full + kRing;                         // [kRing]
    uint64_t* acc_full = empty + kRing;                     // [2]
    uint64_t* acc_empty = acc_full + 2;                     // [2]
    uint64_t* act_ready = acc_empty + 2;                    // [1]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(act_ready + 1);
    volatile uint32_t* abort_flag = tmem_slot + 1;
    uint32_t* last_flag = tmem_slot + 2;
    float* red = reinterpret_cast<float*>(tmem_slot + 4);   // [4]
    float* col_scale = red + 4;                              // [kCols]

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t split = blockIdx.x % p.splits;
    const uint32_t group = blockIdx.x / p.splits, groups = gridDim.x / p.splits;
    const uint32_t stage0 = split * p.per;
    const uint32_t stage1 = min(p.k_stages, stage0 + p.per);
    const uint32_t k_bytes = p.k / 2;

    if (threadIdx.x == 0) {
        for (uint32_t i = 0; i < kRing; ++i) {
            umma::mbar_init(&full[i], 1);
            umma::mbar_init(&empty[i], 1);
        }
        for (uint32_t i = 0; i < 2; ++i) {
            umma::mbar_init(&acc_full[i], 1);
            umma::mbar_init(&acc_empty[i], 4);
        }
        umma::mbar_init(act_ready, 1);
        *abort_flag = 0;
        *last_flag = 0;
        umma::fence_barrier_init();
        umma::prefetch_tensormap(&map_w);
    }
    if (warp == 1) {
        umma::tmem_alloc(tmem_slot, kTmemCols);
        umma::tmem_relinquish();
    }
    umma::tc_fence_before();
    __syncthreads();
    umma::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---------------------------------------------------------------- weight producer
        const bool leader = umma::elect_one();
        uint32_t it = 0;
        bool ok = true;
        for (uint32_t rt = group; ok && rt < p.row_tiles; rt += groups) {
            const uint8_t* sf_base = p.sf_w + static_cast<size_t>(rt) * p.sf_tile_stride;
            for (uint32_t s = stage0; s < stage1; ++s, ++it) {
                const uint32_t slot = it % kRing, phase = (it / kRing) & 1;
                if (!__all_sync(0xffffffffu, umma::mbar_wait(&empty[slot], phase ^ 1, abort_flag, p.status, umma::kTimeoutEmpty))) { ok = false; break; }
                if (leader) {
                    const uint32_t kb = min(4u, (k_bytes - s * kStageK + 31) / 32);
                    umma::mbar_arrive_expect_tx(&full[slot], kWeightTile + kb * 512);
                    umma::tma_load_2d(ring_w + slot * kWeightTile, &map_w, &full[slot], static_cast<int32_t>(s * kStageK),
                                      static_cast<int32_t>(rt * kRows));
                    umma::bulk_load_1d(ring_sf + slot * kSfTile, sf_base + static_cast<size_t>(s) * kSfTile, kb * 512, &full[slot]);
                }
                __syncwarp();
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issuer
        const bool leader = umma::elect_one();
        constexpr uint32_t idesc = umma::idesc_nvf4(kCols);
        const uint32_t w_lo0 = umma::desc_lo_sw128(umma::smem_u32(ring_w));
        const uint32_t a_lo0 = umma::desc_lo_sw128(umma::smem_u32(act));
        const uint32_t wsf_lo0 = umma::desc_lo_scales(umma::smem_u32(ring_sf));
        const uint32_t asf_lo0 = umma::desc_lo_scales(umma::smem_u32(act_sf));
        const uint32_t sfw_tmem = tmem_base + 32, sfa_tmem = tmem_base + 48;
        const uint32_t tail_kb = ((k_bytes - (p.k_stages - 1) * kStageK) + 31) / 32;
        bool ok = __all_sync(0xffffffffu, umma::mbar_wait(act_ready, 0, abort_flag, p.status, umma::kTimeoutOther));
        umma::tc_fence_after();
        uint32_t it = 0, tile = 0;
        for (uint32_t rt = group; ok && rt < p.row_tiles; rt += groups, ++tile) {
            const uint32_t acc = tile & 1, acc_phase = (tile >> 1) & 1;
            if (!__all_sync(0xffffffffu, umma::mbar_wait(&acc_empty[acc], acc_phase ^ 1, abort_flag, p.status, umma::kTimeoutTmemEmpty))) { ok = false; break; }
            umma::tc_fence_after();
            const uint32_t d_tmem = tmem_base + acc * kCols;
            for (uint32_t s = stage0; s < stage1; ++s, ++it) {
                const uint32_t slot = it % kRing, phase = (it / kRing) & 1;
                if (!__all_sync(0xffffffffu, umma::mbar_wait(&full[slot], phase, abort_flag, p.status, umma::kTimeoutFull))) { ok = false; break; }
                umma::tc_fence_after();
                if (leader) {
                    const uint32_t ls = s - stage0;
                    const uint32_t w_lo = w_lo0 + slot * (kWeightTile >> 4), a_lo = a_lo0 + ls * (kActTile >> 4);
                    const uint32_t wsf_lo = wsf_lo0 + slot * (kSfTile >> 4), asf_lo = asf_lo0 + ls * (kSfTile >> 4);
                    const uint32_t kb = (s + 1 < p.k_stages) ? 4u : tail_kb;
                    for (uint32_t j = 0; j < kb; ++j) {
                        umma::tc_copy_scales(sfw_tmem + j * 4, umma::make_desc(wsf_lo + j * 32, umma::kDescHiScales));
                        umma::tc_copy_scales(sfa_tmem + j * 4, umma::make_desc(asf_lo + j * 32, umma::kDescHiScales));
                    }
                    for (uint32_t j = 0; j < kb; ++j)
                        umma::mma_nvf4(d_tmem, umma::make_desc(w_lo + j * 2, umma::kDescHiSw128),
                                       umma::make_desc(a_lo + j * 2, umma::kDescHiSw128), idesc, sfw_tmem + j * 4, sfa_tmem + j * 4,
                                       (s > stage0 || j > 0) ? 1u : 0u);
                    umma::tc_commit(&empty[slot]);
                }
                __syncwarp();
            }
            if (ok && leader) umma::tc_commit(&acc_full[acc]);
            __syncwarp();
        }
    } else {
        // ---------------------------------------------------------------- activation expansion, then epilogue
        const uint32_t te = threadIdx.x - 64;  // 0..127
        const uint32_t quad = warp & 3;
        // zero the resident activation tiles and their scales (rows past tokens * TERMS and the K tail stay zero)
        {
            uint4* z = reinterpret_cast<uint4*>(act);
            for (uint32_t i = te; i < kMaxLocalStages * kActTile / 16; i += 128) z[i] = make_uint4(0, 0, 0, 0);
            z = reinterpret_cast<uint4*>(act_sf);
            for (uint32_t i = te; i < kMaxLocalStages * kSfTile / 16; i += 128) z[i] = make_uint4(0, 0, 0, 0);
            if (te < kCols) col_scale[te] = 0.0f;
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        const uint32_t k_begin = stage0 * 256, k_end = min(p.k, stage1 * 256);
        const uint32_t nblk = k_end > k_begin ? (k_end - k_begin) / 16 : 0;
        for (uint32_t m = 0; m < p.tokens; ++m) {
            float r[16];
            float amax = 0.0f;
            if (te < nblk) {
                load16<XT>(static_cast<const XT*>(p.x) + static_cast<size_t>(m) * p.k + k_begin + te * 16, r);
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    if (!(fabsf(r[i]) < __int_as_float(0x7f800000))) r[i] = 0.0f;
                    amax = fmaxf(amax, fabsf(r[i]));
                }
            } else {
#pragma unroll
                for (int i = 0; i < 16; ++i) r[i] = 0.0f;
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
            if (lane == 0) red[quad] = amax;
            asm volatile("bar.sync 1, 128;" ::: "memory");
            amax = fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3]));
            asm volatile("bar.sync 1, 128;" ::: "memory");
            float g = amax == 0.0f ? 1.0f : amax * (1.0f / kRowScaleDivisor);
#pragma unroll 1
            for (uint32_t j = 0; j < TERMS; ++j) {
                const uint32_t row = m * TERMS + j;
                if (te == 0) col_scale[row] = g;
                if (te < nblk) {
                    const float inv_g = __frcp_rn(g);
                    float bmax = 0.0f;
#pragma unroll
                    for (int i = 0; i < 16; ++i) bmax = fmaxf(bmax, fabsf(r[i] * inv_g));
                    const uint8_t sc = bmax == 0.0f ? 0 : ue4m3_code(bmax * (1.0f / 6.0f));
                    const float sv = e4m3_value(sc);
                    const float inv = sv == 0.0f ? 0.0f : __frcp_rn(sv) * inv_g;
                    const float back = sv * g;
                    uint32_t w[2] = {0u, 0u};
#pragma unroll
                    for (int i = 0; i < 16; i += 2) {
                        const uint32_t byte = e2m1x2_code(r[i] * inv, r[i + 1] * inv);
                        w[i / 8] |= byte << ((i % 8) * 4);
                        r[i] = fmaf(-e2m1_value(byte & 0xfu), back, r[i]);
                        r[i + 1] = fmaf(-e2m1_value(byte >> 4), back, r[i + 1]);
                    }
                    // block te of the slice: stage te / 16, 16-byte chunk (te % 16) / 2 (XOR-swizzled by the row), half te % 2
                    const uint32_t ls = te >> 4, chunk = (te & 15) >> 1, half = te & 1;
                    uint8_t* dst = act + ls * kActTile + row * 128 + ((chunk ^ (row & 7)) << 4) + half * 8;
                    *reinterpret_cast<uint2*>(dst) = make_uint2(w[0], w[1]);
                    // scale byte: 512-byte tile per 64 elements, [row % 32][row / 32][block % 4]
                    act_sf[ls * kSfTile + ((te & 15) >> 2) * 512 + (row & 31) * 16 + (row >> 5) * 4 + (te & 3)] = sc;
                }
                g *= 0.25f;
            }
        }
        umma::fence_proxy_async();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (te == 0) umma::mbar_arrive(act_ready);

        uint32_t tile = 0;
        bool ok = true;
        const uint32_t padded_rows = p.row_tiles * kRows;
        for (uint32_t rt = group; ok && rt < p.row_tiles; rt += groups, ++tile) {
            const uint32_t acc = tile & 1, acc_phase = (tile >> 1) & 1;
            if (!umma::mbar_wait(&acc_full[acc], acc_phase, abort_flag, p.status, umma::kTimeoutTmemFull)) { ok = false; break; }
            umma::tc_fence_after();
            uint32_t raw[16];
            if (stage0 < stage1) {
                umma::tmem_load_32x16(tmem_base + ((quad * 32) << 16) + acc * kCols, raw);
                umma::tmem_load_wait();
            } else {
#pragma unroll
                for (int i = 0; i < 16; ++i) raw[i] = 0;
            }
            umma::tc_fence_before();
            __syncwarp();
            if (lane == 0) umma::mbar_arrive(&acc_empty[acc]);
            const uint32_t row = rt * kRows + quad * 32 + lane;
            const bool row_ok = row < p.n;
            float part[kCols / TERMS];
#pragma unroll
            for (int m = 0; m < static_cast<int>(kCols / TERMS); ++m) {
                float sum = 0.0f;
#pragma unroll
                for (int j = 0; j < TERMS; ++j) sum = fmaf(__uint_as_float(raw[m * TERMS + j]), col_scale[m * TERMS + j], sum);
                part[m] = sum;
            }
            auto emit = [&](uint32_t m, float sum) {
                const size_t index = static_cast<size_t>(m) * p.ld_out + row;
                float v = sum * p.alpha;
                if (p.beta != 0.0f && p.c_in)
                    v = fmaf(p.beta, p.out_is_bf16 ? bf16_bits_to_float(static_cast<const uint16_t*>(p.c_in)[index])
                                                   : static_cast<const float*>(p.c_in)[index], v);
                if (p.out_is_bf16) static_cast<uint16_t*>(p.out)[index] = float_to_bf16_bits(v);
                else static_cast<float*>(p.out)[index] = v;
            };
            if (p.splits == 1) {
                if (row_ok)
#pragma unroll
                    for (int m = 0; m < static_cast<int>(kCols / TERMS); ++m)
                        if (static_cast<uint32_t>(m) < p.tokens) emit(m, part[m]);
            } else {
#pragma unroll
                for (int m = 0; m < static_cast<int>(kCols / TERMS); ++m)
                    if (static_cast<uint32_t>(m) < p.tokens)
                        p.workspace[(static_cast<size_t>(split) * p.tokens + m) * padded_rows + row] = part[m];
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
                    if (row_ok)
                        for (uint32_t m = 0; m < p.tokens; ++m) {
                            float sum = 0.0f;
                            for (uint32_t s = 0; s < p.splits; ++s)
                                sum += __ldcg(&p.workspace[(static_cast<size_t>(s) * p.tokens + m) * padded_rows + row]);
                            emit(m, sum);
                        }
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");
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

}  // namespace decode
}  // namespace eider
