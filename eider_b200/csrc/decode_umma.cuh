// Single-launch NVFP4 W4A16 decode GEMV for one or two tokens (tcgen05).
//
// The weight matrix is the only thing that moves: 128 output features x 128 bytes of K per stage stream through a
// deep TMA ring straight into the tensor cores.  The activation never goes through global memory in quantized form:
// each CTA owns one K split (fixed for the whole launch), and its four epilogue warps expand that slice of x into
// residual NVFP4 terms (x ~= sum_j g_j deq(q_j), g_j = g_0 / 4^j, g_0 from the slice maximum) directly into
// shared-memory operand tiles in the 128-byte-swizzled K-major layout the MMA descriptors expect, while the producer
// warp is already prefetching weights.  Partial sums of the K splits meet in a small fp32 scratch; the last CTA of a
// row tile reduces them in split order.
//
// PREPARED variant: the producer of x has already written the residual terms in the operand layout (rows of packed codes,
// scale bytes as [64-element block][operand row][16 bytes], one power-of-two scale per row).  Nothing is expanded and no
// slice stays resident: every ring slot holds a weight stage and the matching operand stage (one tiled TMA load and one
// bulk copy of scale bytes), the operand half being requested only once the kernel before this one has finished.  Up to
// eight bf16 tokens (32 operand rows) share the launch.
#pragma once

#include <cuda.h>

#include "common.cuh"
#include "umma.cuh"

namespace eider {
namespace decode {

constexpr uint32_t kRows = 128;          // output features per tile (MMA M)
constexpr uint32_t kCols = 16;           // MMA N of the expanding variant: tokens x terms, zero padded (32 for wide prepared operands)
constexpr uint32_t kStageK = 128;        // bytes of K per stage
constexpr uint32_t kMaxLocalStages = 20; // stages of one K split (its activation slice stays resident): 20 * 256 elements
constexpr uint32_t kMaxRing = 12;        // weight stages in flight (the host picks how many fit beside the resident slice)
constexpr uint32_t kMaxExpandThreads = 640;  // one thread per 8 activation elements of the slice
constexpr uint32_t kWeightTile = kRows * kStageK;  // 16 KB
constexpr uint32_t kSfTile = 4 * 512;              // scales of one stage for 128 rows
constexpr uint32_t kSmemBytes = 226 * 1024;        // whole carve-out; ring depth = what is left beside the resident slice
constexpr uint32_t kFixedBytes = 1024 /*alignment*/ + 256 /*scale window overrun*/ + 512 /*barriers, flags*/;
// operand rows (MMA N) -> bytes of one stage of the resident activation slice: the tile and its scale bytes (per 64 elements
// [row][16 bytes], of which the first four are the row's four block scales)
__host__ __device__ constexpr uint32_t act_tile_bytes(uint32_t cols) { return cols * kStageK; }
__host__ __device__ constexpr uint32_t act_sf_stage_bytes(uint32_t cols) { return 4 * cols * 16; }
__host__ __device__ inline uint32_t ring_depth(uint32_t per, uint32_t cols = kCols) {
    const uint32_t left = kSmemBytes - kFixedBytes - per * (act_tile_bytes(cols) + act_sf_stage_bytes(cols));
    const uint32_t r = left / (kWeightTile + kSfTile);
    return r > kMaxRing ? kMaxRing : r;
}
// tensor memory: two accumulators of COLS columns, 16 + 16 scale columns
__host__ __device__ constexpr uint32_t tmem_cols(uint32_t cols) { return 2 * cols + 32 <= 64 ? 64 : 128; }

struct Params {
    const void* x;            // [tokens][k] bf16 or f32 (expanding variant)
    const uint8_t* x_sf;      // prepared variant: scale bytes [k / 64][COLS][16]
    const float* x_col_scale; // prepared variant: [COLS] power-of-two scale of every operand row
    uint32_t tokens, n, k;
    uint32_t k_stages;        // ceil(k / 256)
    uint32_t splits, per;     // K splits and stages per split (per <= kMaxLocalStages)
    uint32_t ring;            // weight stages in flight = ring_depth(per)
    uint32_t expand_threads;  // multiple of 32, >= 128: threads 64 .. 64 + expand_threads
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
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const float4 f = __ldg(reinterpret_cast<const float4*>(p) + h);
        v[4 * h] = f.x; v[4 * h + 1] = f.y; v[4 * h + 2] = f.z; v[4 * h + 3] = f.w;
    }
}

// Decodes through the conversion instructions (the expansion only needs x ~= sum of terms, not the oracle's bit pattern).
__device__ __forceinline__ float fast_e4m3(uint8_t code) {
    const __half2_raw h = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(code), __NV_E4M3);
    return __half2float(__half(__half_raw{h.x}));
}
__device__ __forceinline__ float2 fast_e2m1x2(uint32_t byte) {
    const __half2_raw h = __nv_cvt_fp4x2_to_halfraw2(static_cast<__nv_fp4x2_storage_t>(byte), __NV_E2M1);
    return make_float2(__half2float(__half(__half_raw{h.x})), __half2float(__half(__half_raw{h.y})));
}

template <int TERMS, typename XT, int COLS = kCols, bool PREPARED = false>
__global__ void __launch_bounds__(PREPARED ? 192 : 64 + kMaxExpandThreads, PREPARED ? 3 : 1) nvfp4_decode_fused_kernel(const __grid_constant__ CUtensorMap map_w,
                                                                                      const __grid_constant__ CUtensorMap map_x, const Params p) {
    constexpr uint32_t kActTile = act_tile_bytes(COLS);
    constexpr uint32_t kActSfStage = act_sf_stage_bytes(COLS);
    constexpr uint32_t kTmemCols = tmem_cols(COLS);
    static_assert(PREPARED || COLS == kCols, "the expanding variant writes 16 operand rows");
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    const uint32_t kRing = p.ring;
    uint8_t* ring_w = smem;
    const uint32_t act_slots = PREPARED ? kRing : p.per;    // operand stages in shared memory: the ring's, or the CTA's whole slice
    uint8_t* act = ring_w + kRing * kWeightTile;            // [act_slots][COLS rows][128 B], swizzled
    uint8_t* ring_sf = act + act_slots * kActTile;          // [ring][2 KB]
    uint8_t* act_sf = ring_sf + kRing * kSfTile;            // [act_slots][4][COLS rows][16 B] (+ 256 bytes the last copy window overruns)
    uint8_t* tail = act_sf + act_slots * kActSfStage + 256;
    uint64_t* full = reinterpret_cast<uint64_t*>(tail);     // [kMaxRing]
    uint64_t* empty = full + kMaxRing;                      // [kMaxRing]
    uint64_t* acc_full = empty + kMaxRing;                  // [2]
    uint64_t* acc_empty = acc_full + 2;                     // [2]
    uint64_t* act_ready = acc_empty + 2;                    // [1]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(act_ready + 1);
    volatile uint32_t* abort_flag = tmem_slot + 1;
    uint32_t* last_flag = tmem_slot + 2;
    float* red = reinterpret_cast<float*>(tmem_slot + 4);   // [32]
    float* col_scale = red + 32;                              // [COLS <= 32]

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t split = blockIdx.x % p.splits;
    const uint32_t group = blockIdx.x / p.splits, groups = gridDim.x / p.splits;
    const uint32_t stage0 = split * p.per;
    const uint32_t stage1 = min(p.k_stages, stage0 + p.per);
    const uint32_t k_bytes = p.k / 2;

    // The expansion warps clear their operand tiles before the CTA-wide setup barrier.  Under a programmatic dependent
    // launch everything up to griddepcontrol.wait (setup, the first weight stages) overlaps the tail of the kernel that
    // ran before; x, the split-K scratch and the output are only touched after the wait.
    const uint32_t k_begin = stage0 * 256, k_end = min(p.k, stage1 * 256);
    const uint32_t nhalf = k_end > k_begin ? (k_end - k_begin) / 8 : 0;  // 8-element half blocks, one per expansion thread
    if (warp >= 2) {
        const uint32_t te = threadIdx.x - 64;
        uint4* z = reinterpret_cast<uint4*>(act);
        if constexpr (!PREPARED)  // (the tiled loads of the prepared variant write whole tiles, zero past the end of K)
            for (uint32_t i = te; i < p.per * kActTile / 16; i += p.expand_threads) z[i] = make_uint4(0, 0, 0, 0);
        z = reinterpret_cast<uint4*>(act_sf);  // (prepared: a K tail copies fewer scale bytes than a slot holds; the rest stays finite)
        for (uint32_t i = te; i < (act_slots * kActSfStage + 256) / 16; i += p.expand_threads) z[i] = make_uint4(0, 0, 0, 0);
        if (te < COLS) col_scale[te] = 0.0f;
    }
    if (threadIdx.x == 0) {
        for (uint32_t i = 0; i < kMaxRing; ++i) {
            umma::mbar_init(&full[i], PREPARED ? 2 : 1);  // prepared: the weight half and the operand half arrive separately
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
        if constexpr (PREPARED) umma::prefetch_tensormap(&map_x);
    }
    auto load_stage = [&](uint32_t rt, uint32_t s, uint32_t slot) {
        const uint8_t* sf_base = p.sf_w + static_cast<size_t>(rt) * p.sf_tile_stride;
        const uint32_t kb = min(4u, (k_bytes - s * kStageK + 31) / 32);
        umma::mbar_arrive_expect_tx(&full[slot], kWeightTile + kb * 512);
        umma::tma_load_2d(ring_w + slot * kWeightTile, &map_w, &full[slot], static_cast<int32_t>(s * kStageK), static_cast<int32_t>(rt * kRows));
        umma::bulk_load_1d(ring_sf + slot * kSfTile, sf_base + static_cast<size_t>(s) * kSfTile, kb * 512, &full[slot]);
    };
    auto load_operand = [&](uint32_t s, uint32_t slot) {  // prepared variant: stage s of the operand into ring slot `slot`
        const uint32_t blocks = min(4u, (p.k + 63) / 64 - s * 4);
        umma::mbar_arrive_expect_tx(&full[slot], kActTile + blocks * COLS * 16);
        umma::tma_load_2d(act + slot * kActTile, &map_x, &full[slot], static_cast<int32_t>(s * kStageK), 0);
        umma::bulk_load_1d(act_sf + slot * kActSfStage, p.x_sf + static_cast<size_t>(s) * 4 * COLS * 16, blocks * COLS * 16, &full[slot]);
    };
    // The first ring of weight stages of the first row tile is requested by the thread that initialised the barriers,
    // before the setup barrier: weights depend on nothing, and every slot is free.
    uint32_t early = 0;
    if (group < p.row_tiles) early = min(kRing, stage1 > stage0 ? stage1 - stage0 : 0u);
    if (threadIdx.x == 0)
        for (uint32_t i = 0; i < early; ++i) load_stage(group, stage0 + i, i);
    if (warp == 1) {
        umma::tmem_alloc(tmem_slot, kTmemCols);
        umma::tmem_relinquish();
    }
    umma::tc_fence_before();
    __syncthreads();
    umma::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    if (threadIdx.x == 0) {
        umma::griddep_launch_dependents();  // the next kernel in the stream may start its own setup and weight requests
    }

    if (warp == 0) {
        // ---------------------------------------------------------------- weight producer
        const bool leader = umma::elect_one();
        uint32_t it = 0;
        bool ok = true;
        if constexpr (PREPARED) {
            // the operand is the output of the kernel before this one; the early weight stages get their operand halves now
            umma::griddep_wait();
            if (leader) {
                umma::fence_proxy_async();  // the cleared scale bytes are ordered before the copies that overwrite them
                for (uint32_t i = 0; i < early; ++i) load_operand(stage0 + i, i);
            }
            __syncwarp();
        }
        for (uint32_t rt = group; ok && rt < p.row_tiles; rt += groups) {
            for (uint32_t s = stage0; s < stage1; ++s, ++it) {
                if (it < early) continue;  // requested before the setup barrier (by lane 0, the same thread order as here)
                const uint32_t slot = it % kRing, phase = (it / kRing) & 1;
                if (!__all_sync(0xffffffffu, umma::mbar_wait(&empty[slot], phase ^ 1, abort_flag, p.status, umma::kTimeoutEmpty))) { ok = false; break; }
                if (leader) {
                    load_stage(rt, s, slot);
                    if constexpr (PREPARED) load_operand(s, slot);
                }
                __syncwarp();
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issuer
        const bool leader = umma::elect_one();
        constexpr uint32_t idesc = umma::idesc_nvf4(COLS);
        const uint32_t w_lo0 = umma::desc_lo_sw128(umma::smem_u32(ring_w));
        const uint32_t a_lo0 = umma::desc_lo_sw128(umma::smem_u32(act));
        const uint32_t wsf_lo0 = umma::desc_lo_scales(umma::smem_u32(ring_sf));
        const uint32_t asf_lo0 = umma::desc_lo_scales(umma::smem_u32(act_sf));
        const uint32_t sfw_tmem = tmem_base + 2 * COLS, sfa_tmem = tmem_base + 2 * COLS + 16;
        const uint32_t tail_kb = ((k_bytes - (p.k_stages - 1) * kStageK) + 31) / 32;
        bool ok = PREPARED || __all_sync(0xffffffffu, umma::mbar_wait(act_ready, 0, abort_flag, p.status, umma::kTimeoutOther));
        umma::tc_fence_after();
        uint32_t it = 0, tile = 0;
        for (uint32_t rt = group; ok && rt < p.row_tiles; rt += groups, ++tile) {
            const uint32_t acc = tile & 1, acc_phase = (tile >> 1) & 1;
            if (!__all_sync(0xffffffffu, umma::mbar_wait(&acc_empty[acc], acc_phase ^ 1, abort_flag, p.status, umma::kTimeoutTmemEmpty))) { ok = false; break; }
            umma::tc_fence_after();
            const uint32_t d_tmem = tmem_base + acc * COLS;
            for (uint32_t s = stage0; s < stage1; ++s, ++it) {
                const uint32_t slot = it % kRing, phase = (it / kRing) & 1;
                if (!__all_sync(0xffffffffu, umma::mbar_wait(&full[slot], phase, abort_flag, p.status, umma::kTimeoutFull))) { ok = false; break; }
                umma::tc_fence_after();
                if (leader) {
                    const uint32_t ls = PREPARED ? slot : s - stage0;  // where the operand stage sits
                    const uint32_t w_lo = w_lo0 + slot * (kWeightTile >> 4), a_lo = a_lo0 + ls * (kActTile >> 4);
                    const uint32_t wsf_lo = wsf_lo0 + slot * (kSfTile >> 4), asf_lo = asf_lo0 + ls * (kActSfStage >> 4);
                    const uint32_t first = s > stage0 ? 1u : 0u;
                    if (s + 1 < p.k_stages || tail_kb == 4) {
#pragma unroll
                        for (uint32_t j = 0; j < 4; ++j) {
                            umma::tc_copy_scales(sfw_tmem + j * 4, umma::make_desc(wsf_lo + j * 32, umma::kDescHiScales));
                            umma::tc_copy_scales(sfa_tmem + j * 4, umma::make_desc(asf_lo + j * COLS, umma::kDescHiScales));
                        }
#pragma unroll
                        for (uint32_t j = 0; j < 4; ++j)
                            umma::mma_nvf4(d_tmem, umma::make_desc(w_lo + j * 2, umma::kDescHiSw128),
                                           umma::make_desc(a_lo + j * 2, umma::kDescHiSw128), idesc, sfw_tmem + j * 4,
                                           sfa_tmem + j * 4, j == 0 ? first : 1u);
                    } else {
                        for (uint32_t j = 0; j < tail_kb; ++j) {
                            umma::tc_copy_scales(sfw_tmem + j * 4, umma::make_desc(wsf_lo + j * 32, umma::kDescHiScales));
                            umma::tc_copy_scales(sfa_tmem + j * 4, umma::make_desc(asf_lo + j * COLS, umma::kDescHiScales));
                        }
                        for (uint32_t j = 0; j < tail_kb; ++j)
                            umma::mma_nvf4(d_tmem, umma::make_desc(w_lo + j * 2, umma::kDescHiSw128),
                                           umma::make_desc(a_lo + j * 2, umma::kDescHiSw128), idesc, sfw_tmem + j * 4,
                                           sfa_tmem + j * 4, j == 0 ? first : 1u);
                    }
                    umma::tc_commit(&empty[slot]);
                }
                __syncwarp();
            }
            if (ok && leader) umma::tc_commit(&acc_full[acc]);
            __syncwarp();
        }
    } else {
        // ---------------------------------------------------------------- activation expansion, then epilogue
        const uint32_t te = threadIdx.x - 64;  // 0 .. expand_threads - 1; the first 128 go on to be the epilogue
        const uint32_t quad = warp & 3;
        umma::griddep_wait();  // x may be the previous kernel's output; scratch, counters and the output are shared with it
        if constexpr (PREPARED) {
            // (the producer warp requests the operand stages; the epilogue only needs the row scales)
            if (te < COLS) col_scale[te] = __ldg(p.x_col_scale + te);
            asm volatile("bar.sync 1, %0;" ::"r"(p.expand_threads) : "memory");
        } else {
        // (operand tiles were cleared before the setup barrier: rows past tokens * TERMS and the K tail stay zero)
        for (uint32_t m = 0; m < p.tokens; ++m) {
            float r[8];
            float amax = 0.0f;
            if (te < nhalf) {
                load8<XT>(static_cast<const XT*>(p.x) + static_cast<size_t>(m) * p.k + k_begin + te * 8, r);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    if (!(fabsf(r[i]) < __int_as_float(0x7f800000))) r[i] = 0.0f;
                    amax = fmaxf(amax, fabsf(r[i]));
                }
            } else {
#pragma unroll
                for (int i = 0; i < 8; ++i) r[i] = 0.0f;
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
            if (lane == 0) red[te >> 5] = amax;
            asm volatile("bar.sync 1, %0;" ::"r"(p.expand_threads) : "memory");
            {
                float mx = 0.0f;
                for (uint32_t w = 0; w < p.expand_threads / 32; ++w) mx = fmaxf(mx, red[w]);
                amax = mx;
            }
            asm volatile("bar.sync 1, %0;" ::"r"(p.expand_threads) : "memory");
            float g = row_scale_pow2(amax);
            float inv_g = pow2_reciprocal(g);
            const uint32_t blk = te >> 1, half = te & 1;
            const uint32_t ls = blk >> 4, chunk = (blk & 15) >> 1;
#pragma unroll
            for (uint32_t j = 0; j < TERMS; ++j) {
                const uint32_t row = m * TERMS + j;
                if (te == 0) col_scale[row] = g;
                float bmax = 0.0f;
#pragma unroll
                for (int i = 0; i < 8; ++i) bmax = fmaxf(bmax, fabsf(r[i] * inv_g));
                bmax = fmaxf(bmax, __shfl_xor_sync(0xffffffffu, bmax, 1));  // the other half of the block
                const uint8_t sc = bmax == 0.0f ? 0 : ue4m3_code(bmax * (1.0f / 6.0f));
                const float sv = fast_e4m3(sc);
                const float inv = sv == 0.0f ? 0.0f : __fdividef(inv_g, sv);
                const float back = sv * g;
                uint32_t w = 0;
#pragma unroll
                for (int i = 0; i < 8; i += 2) {
                    const uint32_t byte = e2m1x2_code(r[i] * inv, r[i + 1] * inv);
                    w |= byte << (i * 4);
                    const float2 q = fast_e2m1x2(byte);  // what the tensor core will read back for these two codes
                    r[i] = fmaf(-q.x, back, r[i]);
                    r[i + 1] = fmaf(-q.y, back, r[i + 1]);
                }
                if (te < nhalf) {
                    // block blk of the slice: stage blk / 16, 16-byte chunk (blk % 16) / 2 XOR-swizzled by the row,
                    // 8 bytes per block, 4 per half
                    uint8_t* dst = act + ls * kActTile + row * 128 + ((chunk ^ (row & 7)) << 4) + (blk & 1) * 8 + half * 4;
                    *reinterpret_cast<uint32_t*>(dst) = w;
                    // scale byte: 256 bytes per 64 elements, [row < 16][16 bytes, the first four = block % 4]; the 512-byte copy
                    // window of the next group overlaps it, the extra rows feed MMA columns that do not exist
                    if (half == 0) act_sf[ls * kActSfStage + ((blk & 15) >> 2) * 256 + row * 16 + (blk & 3)] = sc;
                }
                g *= 0.25f;
                inv_g *= 4.0f;
            }
        }
        umma::fence_proxy_async();
        asm volatile("bar.sync 1, %0;" ::"r"(p.expand_threads) : "memory");
        if (te == 0) umma::mbar_arrive(act_ready);
        }
        if (te >= 128) goto teardown;  // the extra expansion warps are done

        uint32_t tile = 0;
        bool ok = true;
        const uint32_t padded_rows = p.row_tiles * kRows;
        for (uint32_t rt = group; ok && rt < p.row_tiles; rt += groups, ++tile) {
            const uint32_t acc = tile & 1, acc_phase = (tile >> 1) & 1;
            if (!umma::mbar_wait(&acc_full[acc], acc_phase, abort_flag, p.status, umma::kTimeoutTmemFull)) { ok = false; break; }
            umma::tc_fence_after();
            uint32_t raw[COLS];
            if (stage0 < stage1) {
                if constexpr (COLS == 16) umma::tmem_load_32x16(tmem_base + ((quad * 32) << 16) + acc * COLS, *reinterpret_cast<uint32_t(*)[16]>(&raw[0]));
                else umma::tmem_load_32x32(tmem_base + ((quad * 32) << 16) + acc * COLS, *reinterpret_cast<uint32_t(*)[32]>(&raw[0]));
                umma::tmem_load_wait();
            } else {
#pragma unroll
                for (int i = 0; i < COLS; ++i) raw[i] = 0;
            }
            umma::tc_fence_before();
            __syncwarp();
            if (lane == 0) umma::mbar_arrive(&acc_empty[acc]);
            const uint32_t row = rt * kRows + quad * 32 + lane;
            const bool row_ok = row < p.n;
            float part[COLS / TERMS];
#pragma unroll
            for (int m = 0; m < static_cast<int>(COLS / TERMS); ++m) {
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
                    for (int m = 0; m < static_cast<int>(COLS / TERMS); ++m)
                        if (static_cast<uint32_t>(m) < p.tokens) emit(m, part[m]);
            } else {
#pragma unroll
                for (int m = 0; m < static_cast<int>(COLS / TERMS); ++m)
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
                    if (row_ok) {
                        // the partials of every token and of four splits at a time are requested before any is used (one
                        // memory round trip per group of splits, not per token); each token is summed in split order
                        constexpr int kTok = COLS / TERMS;
                        float sum[kTok];
#pragma unroll
                        for (int m = 0; m < kTok; ++m) sum[m] = 0.0f;
                        constexpr uint32_t kChunk = kTok <= 4 ? 8 : 4;  // splits per round trip: at most 32 loads in flight
                        for (uint32_t s0 = 0; s0 < p.splits; s0 += kChunk) {
                            float v[kTok][kChunk];
#pragma unroll
                            for (int m = 0; m < kTok; ++m)
#pragma unroll
                                for (uint32_t u = 0; u < kChunk; ++u)
                                    v[m][u] = (static_cast<uint32_t>(m) < p.tokens && s0 + u < p.splits)
                                                  ? __ldcg(&p.workspace[(static_cast<size_t>(s0 + u) * p.tokens + m) * padded_rows + row])
                                                  : 0.0f;
#pragma unroll
                            for (int m = 0; m < kTok; ++m)
#pragma unroll
                                for (uint32_t u = 0; u < kChunk; ++u) sum[m] += v[m][u];
                        }
#pragma unroll
                        for (int m = 0; m < kTok; ++m)
                            if (static_cast<uint32_t>(m) < p.tokens) emit(m, sum[m]);
                    }
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");
            }
        }
    }
teardown:
    umma::tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        umma::tc_fence_after();
        umma::tmem_dealloc(tmem_base, kTmemCols);
    }
}

}  // namespace decode
}  // namespace eider
