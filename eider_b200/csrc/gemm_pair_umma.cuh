// Dense prefill GEMM on CTA pairs: a cluster of two CTAs computes one 256 x 256 output tile with
// tcgen05.mma.cta_group::2.  Each CTA loads its own 128 activation rows, its own activation scale tile and
// only HALF of the 256 weight rows of the tile (the tensor cores of both SMs read both halves), so the
// shared-memory fill traffic per output tile drops from 54 KB to 38 KB per stage and CTA compared with the
// one-CTA kernel, which is what bounds that kernel on large prefill shapes.
//
// Roles per CTA (192 threads, as in the one-CTA kernel):
//   warp 0      TMA producer for this CTA's share of the stage;
//   warp 1      even CTA: issues the scale copies and the MMAs for the pair, and hands stages / accumulators back
//               to BOTH CTAs with tcgen05.commit on each CTA's barrier;
//               odd CTA: forwards "my share of stage s has landed" to the even CTA's full barrier;
//   warps 2..5  epilogue of this CTA's 128 accumulator rows; accumulator hand-back goes to the even CTA.
// Barriers: full[s] of the even CTA counts two arrivals (its own producer and the odd CTA's forwarder) plus its
// own bytes; acc_empty of the even CTA counts the eight epilogue warps of the pair.  Every wait is bounded.
#pragma once

#include "gemm_umma.cuh"

namespace eider {
namespace gemm {

constexpr uint32_t kPairN = 256;      // weight rows per pair tile
constexpr uint32_t kPairHalfN = 128;  // of which each CTA loads half
// The narrow form, 256 x 192 tiles: two whole accumulators fit in tensor memory beside the scale columns (no shared columns
// to hand over between tiles), and a weight matrix of few column tiles divides into more work items (5120 rows: 27 instead
// of 20 for 74 SM pairs).  A tile that does not start on a 128-row scale tile starts two scale columns into it.
constexpr uint32_t kPairNarrowN = 192;

template <int KIND, uint32_t PAIR_N = kPairN> struct PairSmem {
    static constexpr bool kNv = KIND == kNvf4;
    static constexpr uint32_t kA = kTileRows * kStageBytesK;          // this CTA's 128 rows
    static constexpr uint32_t kB = (PAIR_N / 2) * kStageBytesK;       // this CTA's half of the weight rows
    static constexpr uint32_t kSfA = kNv ? 4 * kScaleTileBytes : 0;   // scales of this CTA's rows
    static constexpr uint32_t kSfB = kNv ? 8 * kScaleTileBytes : 0;   // scales of all 256 weight rows
    static constexpr uint32_t kStage = kA + kB + kSfA + kSfB;
    // epilogue staging for TMA stores: per epilogue warp two buffers of 32 rows x 128 bytes (64 bf16 columns)
    static constexpr uint32_t kStoreBuf = 32 * 128;
    static constexpr uint32_t kStore = 4 * 2 * kStoreBuf;
    static constexpr int kStages = (226u * 1024u - kStore) / kStage > 8 ? 8 : static_cast<int>((226u * 1024u - kStore) / kStage);
    static constexpr uint32_t kBytes = kStage * kStages + kStore + 1024 /*alignment slack*/ + 256 /*barriers*/;
};

struct PairTile {
    uint32_t row_tile;  // this CTA's 128-row tile (may be one past the last when the row-tile count is odd)
    uint32_t row0;
    uint32_t col0;      // first weight row of the pair tile
    uint32_t k0, k1;    // K stages of this work item (all of them unless K is split)
    uint32_t split;
};

template <uint32_t PAIR_N = kPairN>
__device__ __forceinline__ bool pair_tile(const Params& p, uint32_t item, uint32_t rank, PairTile& t) {
    const uint32_t row_pairs = (p.row_tiles + 1) / 2;
    if (item >= row_pairs * p.col_tiles * p.splits) return false;
    const uint32_t rp = item % row_pairs;  // row pairs fastest: neighbouring pairs share the weight tile in L2
    const uint32_t rest = item / row_pairs;
    t.row_tile = rp * 2 + rank;
    t.row0 = t.row_tile * kTileRows;
    t.col0 = (rest % p.col_tiles) * PAIR_N;
    t.split = rest / p.col_tiles;
    const uint32_t per = (p.k_stages + p.splits - 1) / p.splits;
    t.k0 = t.split * per;
    t.k1 = min(p.k_stages, t.k0 + per);
    return true;
}

template <int KIND, uint32_t PAIR_N = kPairN>
__global__ void __launch_bounds__(kNumThreads, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap map_rows, const __grid_constant__ CUtensorMap map_cols, const Params p) {
    static_assert(PAIR_N == kPairN || PAIR_N == kPairNarrowN, "pair tiles are 256 or 192 weight rows wide");
    using L = PairSmem<KIND, PAIR_N>;
    using T = TmemPlan<KIND, PAIR_N>;
    constexpr bool kNv = KIND == kNvf4;
    constexpr int STAGES = L::kStages;
    constexpr uint32_t kAcc = T::kAccStages;

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    uint8_t* smem_a = smem;
    uint8_t* smem_b = smem_a + STAGES * L::kA;
    uint8_t* smem_sfa = smem_b + STAGES * L::kB;
    uint8_t* smem_sfb = smem_sfa + STAGES * L::kSfA;
    uint8_t* smem_store = smem + STAGES * L::kStage;  // 1024-byte aligned: the stage size is a multiple of 1024
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem_store + L::kStore);
    uint64_t* full = bars;                    // [STAGES]
    uint64_t* empty = bars + STAGES;          // [STAGES]
    uint64_t* acc_full = bars + 2 * STAGES;   // [kAcc]
    uint64_t* acc_empty = acc_full + kAcc;    // [kAcc] (used in the even CTA)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + kAcc);
    volatile uint32_t* abort_flag = tmem_slot + 1;

    const uint32_t warp = threadIdx.x >> 5;
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t rank = umma::cluster_ctarank();
    const uint32_t pair = blockIdx.x >> 1;
    const uint32_t pairs = gridDim.x >> 1;

    if (threadIdx.x == 0) {
        for (int i = 0; i < STAGES; ++i) {
            umma::mbar_init(&full[i], rank == 0 ? 2 : 1);
            umma::mbar_init(&empty[i], 1);
        }
        for (uint32_t i = 0; i < kAcc; ++i) {
            umma::mbar_init(&acc_full[i], 1);
            umma::mbar_init(&acc_empty[i], 8);  // four epilogue warps in each CTA
        }
        *abort_flag = 0;
        umma::fence_barrier_init();
        umma::prefetch_tensormap(&map_rows);
        umma::prefetch_tensormap(&map_cols);
    }
    if (warp == 1) {
        umma::tmem_alloc_pair(tmem_slot, T::kAlloc);
        umma::tmem_relinquish_pair();
    }
    umma::tc_fence_before();
    __syncthreads();
    umma::cluster_sync_all();  // the other CTA's barriers are initialised before anything arrives on them
    umma::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer (both CTAs)
        const bool leader = umma::elect_one();
        const uint32_t sf_col_tiles = (p.cols + kTileRows - 1) / kTileRows;
        uint32_t it = 0;
        PairTile t;
        bool ok = true;
        bool dep_waited = false;
        for (uint32_t item = pair; ok && pair_tile<PAIR_N>(p, item, rank, t); item += pairs) {
            const bool row_sf = kNv && t.row_tile < p.row_tiles;
            const uint32_t sf_col_tile0 = t.col0 / kTileRows;
            const bool second_sf = sf_col_tile0 + 1 < sf_col_tiles;
            for (uint32_t s = t.k0; s < t.k1; ++s, ++it) {
                const uint32_t stage = it % STAGES;
                const uint32_t phase = (it / STAGES) & 1;
                if (!__all_sync(0xffffffffu, umma::mbar_wait_cluster(&empty[stage], phase ^ 1, abort_flag, p.status, umma::kTimeoutEmpty))) { ok = false; break; }
                if (!leader) continue;
                const uint32_t kb = min(4u, (p.k_bytes - s * kStageBytesK + 31) / 32);  // MMAs in this stage
                uint32_t bytes = L::kA + L::kB;
                if (kNv) bytes += kb * kScaleTileBytes * ((row_sf ? 1 : 0) + 1 + (second_sf ? 1 : 0));
                umma::mbar_arrive_expect_tx(&full[stage], bytes);
                const size_t k_off = static_cast<size_t>(s) * 4 * kScaleTileBytes;
                // weights first: they do not depend on the kernel that ran before this one
                umma::tma_load_2d(smem_b + stage * L::kB, &map_cols, &full[stage], static_cast<int32_t>(s * kStageBytesK),
                                  static_cast<int32_t>(t.col0 + rank * (PAIR_N / 2)));
                if (kNv) {
                    umma::bulk_load_1d(smem_sfb + stage * L::kSfB, p.sf_cols + static_cast<size_t>(sf_col_tile0) * p.sf_tile_stride + k_off,
                                       kb * kScaleTileBytes, &full[stage]);
                    if (second_sf)
                        umma::bulk_load_1d(smem_sfb + stage * L::kSfB + 4 * kScaleTileBytes,
                                           p.sf_cols + static_cast<size_t>(sf_col_tile0 + 1) * p.sf_tile_stride + k_off,
                                           kb * kScaleTileBytes, &full[stage]);
                }
                if (!dep_waited) {
                    umma::griddep_wait();
                    dep_waited = true;
                }
                umma::tma_load_2d(smem_a + stage * L::kA, &map_rows, &full[stage], static_cast<int32_t>(s * kStageBytesK),
                                  static_cast<int32_t>(t.row0));
                if (row_sf)
                    umma::bulk_load_1d(smem_sfa + stage * L::kSfA, p.sf_rows + static_cast<size_t>(t.row_tile) * p.sf_tile_stride + k_off,
                                       kb * kScaleTileBytes, &full[stage]);
            }
        }
    } else if (warp == 1 && rank != 0) {
        // ------------------------------------------------------------------ odd CTA: forward stage arrivals
        const bool leader = umma::elect_one();
        const uint32_t full0_remote = umma::map_to_cta(umma::smem_u32(&full[0]), 0);
        uint32_t it = 0;
        PairTile t;
        bool ok = true;
        for (uint32_t item = pair; ok && pair_tile<PAIR_N>(p, item, rank, t); item += pairs) {
            for (uint32_t s = t.k0; s < t.k1; ++s, ++it) {
                const uint32_t stage = it % STAGES;
                const uint32_t phase = (it / STAGES) & 1;
                if (!__all_sync(0xffffffffu, umma::mbar_wait(&full[stage], phase, abort_flag, p.status, umma::kTimeoutFull))) { ok = false; break; }
                if (leader) umma::mbar_arrive_cluster(full0_remote + stage * 8);
                __syncwarp();
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ even CTA: MMA issuer for the pair
        const bool leader = umma::elect_one();
        constexpr uint32_t idesc = kNv ? umma::idesc_nvf4_pair(PAIR_N) : umma::idesc_f8_pair(PAIR_N);
        const uint32_t a_lo0 = umma::desc_lo_sw128(umma::smem_u32(smem_a));
        const uint32_t b_lo0 = umma::desc_lo_sw128(umma::smem_u32(smem_b));
        const uint32_t sfa_lo0 = umma::desc_lo_scales(umma::smem_u32(smem_sfa));
        const uint32_t sfb_lo0 = umma::desc_lo_scales(umma::smem_u32(smem_sfb));
        const uint32_t sfa_tmem = tmem_base + T::kSfAOffset;
        const uint32_t sfb_tmem = tmem_base + T::kSfBOffset;
        const uint32_t empty0_local = umma::smem_u32(&empty[0]);
        const uint32_t accfull0_local = umma::smem_u32(&acc_full[0]);
        const uint32_t tail_kb = ((p.k_bytes - (p.k_stages - 1) * kStageBytesK) + 31) / 32;  // MMAs in the last stage
        uint32_t it = 0, tile_count = 0;
        PairTile t;
        bool ok = true;
        for (uint32_t item = pair; ok && pair_tile<PAIR_N>(p, item, rank, t); item += pairs, ++tile_count) {
            const uint32_t acc = tile_count % kAcc;
            const uint32_t acc_phase = (tile_count / kAcc) & 1;
            if (!__all_sync(0xffffffffu, umma::mbar_wait_cluster(&acc_empty[acc], acc_phase ^ 1, abort_flag, p.status, umma::kTimeoutTmemEmpty))) { ok = false; break; }
            umma::tc_fence_after();
            const uint32_t d_tmem = tmem_base + (T::kOverlap ? (tile_count & 1) : acc) * T::kAccStride;
            // a column tile that does not start on a 128-row scale tile starts (col0 % 128) / 32 scale columns into it
            const uint32_t sfb_sub = (PAIR_N % kTileRows != 0) ? (t.col0 % kTileRows) / 32 : 0;
            for (uint32_t s = t.k0; s < t.k1; ++s, ++it) {
                const uint32_t stage = it % STAGES;
                const uint32_t phase = (it / STAGES) & 1;
                if (!__all_sync(0xffffffffu, umma::mbar_wait_cluster(&full[stage], phase, abort_flag, p.status, umma::kTimeoutFull))) { ok = false; break; }
                umma::tc_fence_after();
                if (leader) {
                    const uint32_t a_lo = a_lo0 + stage * (L::kA >> 4);
                    const uint32_t b_lo = b_lo0 + stage * (L::kB >> 4);
                    const uint32_t sfa_lo = sfa_lo0 + stage * (L::kSfA >> 4);
                    const uint32_t sfb_lo = sfb_lo0 + stage * (L::kSfB >> 4);
                    const uint32_t nkb = (s + 1 < p.k_stages) ? 4u : tail_kb;
                    if (nkb == 4) {
                        // the scale copies of a 64-element step right in front of its MMA: the copies of step j + 1 then run
                        // under the MMA of step j (measured 1.2 us of 33.9 against all twelve copies first)
#pragma unroll
                        for (uint32_t j = 0; j < 4; ++j) {
                            if (kNv) {
                                umma::tc_copy_scales_pair(sfa_tmem + j * 4, umma::make_desc(sfa_lo + j * 32, umma::kDescHiScales));
                                umma::tc_copy_scales_pair(sfb_tmem + j * 8, umma::make_desc(sfb_lo + j * 32, umma::kDescHiScales));
                                umma::tc_copy_scales_pair(sfb_tmem + j * 8 + 4, umma::make_desc(sfb_lo + (4 + j) * 32, umma::kDescHiScales));
                            }
                            const uint64_t a_desc = umma::make_desc(a_lo + j * 2, umma::kDescHiSw128);
                            const uint64_t b_desc = umma::make_desc(b_lo + j * 2, umma::kDescHiSw128);
                            const uint32_t accumulate = (s > t.k0 || j > 0) ? 1u : 0u;
                            if (kNv) umma::mma_nvf4_pair(d_tmem, a_desc, b_desc, idesc, sfa_tmem + j * 4, sfb_tmem + j * 8 + sfb_sub, accumulate);
                            else umma::mma_f8_pair(d_tmem, a_desc, b_desc, idesc, accumulate);
                        }
                    } else {
                        for (uint32_t j = 0; j < nkb; ++j) {
                            if (kNv) {
                                umma::tc_copy_scales_pair(sfa_tmem + j * 4, umma::make_desc(sfa_lo + j * 32, umma::kDescHiScales));
                                umma::tc_copy_scales_pair(sfb_tmem + j * 8, umma::make_desc(sfb_lo + j * 32, umma::kDescHiScales));
                                umma::tc_copy_scales_pair(sfb_tmem + j * 8 + 4, umma::make_desc(sfb_lo + (4 + j) * 32, umma::kDescHiScales));
                            }
                        }
                        for (uint32_t j = 0; j < nkb; ++j) {
                            const uint64_t a_desc = umma::make_desc(a_lo + j * 2, umma::kDescHiSw128);
                            const uint64_t b_desc = umma::make_desc(b_lo + j * 2, umma::kDescHiSw128);
                            const uint32_t accumulate = (s > t.k0 || j > 0) ? 1u : 0u;
                            if (kNv) umma::mma_nvf4_pair(d_tmem, a_desc, b_desc, idesc, sfa_tmem + j * 4, sfb_tmem + j * 8 + sfb_sub, accumulate);
                            else umma::mma_f8_pair(d_tmem, a_desc, b_desc, idesc, accumulate);
                        }
                    }
                    // the stage is free in both CTAs once these MMAs (and scale copies) retire
                    umma::tc_commit_pair_both(empty0_local + stage * 8);
                }
                __syncwarp();
            }
            if (ok && leader) {
                umma::tc_commit_pair_both(accfull0_local + acc * 8);
            }
            __syncwarp();
        }
    } else {
        // ------------------------------------------------------------------ epilogue warps (both CTAs)
        const uint32_t quad = warp & 3;
        umma::griddep_wait();  // row scales written by the preceding kernel are read below
        const uint32_t accempty0_remote = umma::map_to_cta(umma::smem_u32(&acc_empty[0]), 0);
        uint32_t store_count = 0;  // TMA stores issued by this warp (selects the staging buffer)
        uint32_t tile_count = 0;
        PairTile t;
        bool ok = true;
        for (uint32_t item = pair; ok && pair_tile<PAIR_N>(p, item, rank, t); item += pairs, ++tile_count) {
            const uint32_t acc = tile_count % kAcc;
            const uint32_t acc_phase = (tile_count / kAcc) & 1;
            if (!umma::mbar_wait_cluster(&acc_full[acc], acc_phase, abort_flag, p.status, umma::kTimeoutTmemFull)) { ok = false; break; }
            umma::tc_fence_after();
            const uint32_t row = t.row0 + quad * 32 + lane;
            const bool row_ok = row < p.rows;
            float rs = p.alpha;
            if (p.row_scale && row_ok) rs *= p.row_scale[row];
            const uint32_t buf = T::kOverlap ? (tile_count & 1) : acc;
            const uint32_t taddr = tmem_base + ((quad * 32) << 16) + buf * T::kAccStride;
            // overlapping buffers: buffer 0 shares its last 64 columns, buffer 1 its first ones; drain those first
            auto col_of = [&](uint32_t step) { return (T::kOverlap && buf == 0) ? (PAIR_N - 64 - step * 64) : step * 64; };
            auto issue = [&](uint32_t step, uint32_t (&r)[64]) {
                const uint32_t c = col_of(step);
                umma::tmem_load_32x32(taddr + c, *reinterpret_cast<uint32_t(*)[32]>(&r[0]));
                umma::tmem_load_32x32(taddr + c + 32, *reinterpret_cast<uint32_t(*)[32]>(&r[32]));
            };
            const bool wide = p.out_is_bf16 && (reinterpret_cast<uintptr_t>(p.col_scale) & 15) == 0 && !(p.beta != 0.0f && p.c_in) &&
                              (p.ld_out % 16) == 0 && (reinterpret_cast<uintptr_t>(p.out) & 31) == 0;
            const bool staged = p.out_maps != nullptr;  // (the host sets the maps only for plain bf16 output)
            const bool multicast = p.out_multicast != nullptr;  // (likewise, and only when the column count is a multiple of 8)
            constexpr uint32_t kSteps = PAIR_N / 64;
            uint32_t raw[2][64];
            issue(0, raw[0]);
#pragma unroll
            for (uint32_t step = 0; step < kSteps; ++step) {
                umma::tmem_load_wait();
                if (step + 1 < kSteps) issue(step + 1, raw[(step + 1) & 1]);
                if ((T::kOverlap && step == 0) || (!T::kOverlap && step + 1 == kSteps)) {
                    // (the shared columns of) the accumulator are in registers: the next tile's MMAs may start
                    umma::tc_fence_before();
                    __syncwarp();
                    if (lane == 0) umma::mbar_arrive_cluster(accempty0_remote + acc * 8);
                }
                const uint32_t c = col_of(step);
                if (multicast) {
                    // this warp's 32 rows x 64 columns -> bf16 in the (swizzled) staging buffer, read back so that eight
                    // consecutive lanes cover one row's 128 bytes, and written once through the multicast mapping
                    uint8_t* sbuf = smem_store + quad * 2 * L::kStoreBuf;
                    uint32_t w[32];
                    convert_bf16x64_scaled(&raw[step & 1][0], rs, nullptr, w);
                    const uint32_t row_base = umma::smem_u32(sbuf) + lane * 128;
                    __syncwarp();  // the previous step's read-back is over
#pragma unroll
                    for (uint32_t ch = 0; ch < 8; ++ch)
                        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(row_base + ((ch ^ (lane & 7)) << 4)), "r"(w[4 * ch]),
                                     "r"(w[4 * ch + 1]), "r"(w[4 * ch + 2]), "r"(w[4 * ch + 3])
                                     : "memory");
                    __syncwarp();
                    const uint32_t warp_row0 = t.row0 + quad * 32;
                    const uint32_t ch = lane & 7;
                    const uint32_t col = t.col0 + c + ch * 8;
#pragma unroll
                    for (uint32_t i = 0; i < 8; ++i) {
                        const uint32_t r = i * 4 + (lane >> 3);
                        uint32_t v0, v1, v2, v3;
                        asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v0), "=r"(v1), "=r"(v2), "=r"(v3)
                                     : "r"(umma::smem_u32(sbuf) + r * 128 + ((ch ^ (r & 7)) << 4)) : "memory");
                        if (warp_row0 + r < p.rows && col + 8 <= p.cols)
                            umma::multimem_store_16(static_cast<uint16_t*>(p.out_multicast) + static_cast<size_t>(warp_row0 + r) * p.ld_out + col,
                                                    v0, v1, v2, v3);
                    }
                    continue;
                }
                if (staged) {
                    // this warp's 32 rows x 64 columns -> bf16 in a 128-byte-swizzled staging buffer -> one TMA store per
                    // destination (the hardware clips rows and columns past the end of the output)
                    uint8_t* sbuf = smem_store + (quad * 2 + (store_count & 1)) * L::kStoreBuf;
                    if (store_count >= 2) {
                        if (lane == 0) umma::tma_store_wait_read<1>();  // the stores that last read this buffer have finished reading
                        __syncwarp();
                    }
                    ++store_count;
                    uint32_t w[32];
                    convert_bf16x64_scaled(&raw[step & 1][0], rs, nullptr, w);  // (no column scales on this path: the host checks)
                    const uint32_t row_base = umma::smem_u32(sbuf) + lane * 128;
#pragma unroll
                    for (uint32_t ch = 0; ch < 8; ++ch)
                        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(row_base + ((ch ^ (lane & 7)) << 4)), "r"(w[4 * ch]),
                                     "r"(w[4 * ch + 1]), "r"(w[4 * ch + 2]), "r"(w[4 * ch + 3])
                                     : "memory");
                    umma::fence_proxy_async();
                    __syncwarp();
                    const uint32_t warp_row0 = t.row0 + quad * 32;
                    if (lane == 0) {
                        if (warp_row0 < p.rows && t.col0 + c < p.cols)
                            for (uint32_t q = 0; q < p.n_peers; ++q)
                                umma::tma_store_2d(&p.out_maps[q], sbuf, static_cast<int32_t>(t.col0 + c), static_cast<int32_t>(warp_row0));
                        umma::tma_store_commit();  // one group per use of a staging buffer, empty or not
                    }
                    continue;
                }
                if (!row_ok || t.col0 + c >= p.cols) continue;
                if (p.split_stride != 0) {
                    // split K: this split's unscaled fp32 partial sums (the host sets alpha 1 and no scales on this path)
                    float* dst = static_cast<float*>(p.out) + static_cast<size_t>(t.split) * p.split_stride + static_cast<size_t>(row) * p.ld_out + t.col0 + c;
                    if (t.col0 + c + 64 <= p.cols && (p.ld_out % 4) == 0) {
#pragma unroll
                        for (uint32_t q = 0; q < 16; ++q)
                            reinterpret_cast<float4*>(dst)[q] = make_float4(__uint_as_float(raw[step & 1][4 * q]), __uint_as_float(raw[step & 1][4 * q + 1]),
                                                                            __uint_as_float(raw[step & 1][4 * q + 2]), __uint_as_float(raw[step & 1][4 * q + 3]));
                    } else {
#pragma unroll
                        for (uint32_t i = 0; i < 64; ++i)
                            if (t.col0 + c + i < p.cols) dst[i] = __uint_as_float(raw[step & 1][i]);
                    }
                    continue;
                }
                if (wide && t.col0 + c + 64 <= p.cols) {  // (a tile that hangs over the last column still stores its whole 64-column steps wide)
                    store_row64_all(p, static_cast<size_t>(row) * p.ld_out + t.col0 + c, &raw[step & 1][0], rs,
                                    p.col_scale ? p.col_scale + t.col0 + c : nullptr);
                } else {
#pragma unroll
                    for (uint32_t i = 0; i < 64; ++i) {  // fully unrolled: the accumulator stays in registers
                        const uint32_t col = t.col0 + c + i;
                        if (col >= p.cols) continue;
                        const size_t index = static_cast<size_t>(row) * p.ld_out + col;
                        float x = __uint_as_float(raw[step & 1][i]) * rs;
                        if (p.col_scale) x *= p.col_scale[col];
                        if (p.beta != 0.0f && p.c_in)
                            x = fmaf(p.beta, p.out_is_bf16 ? bf16_bits_to_float(static_cast<const uint16_t*>(p.c_in)[index])
                                                           : static_cast<const float*>(p.c_in)[index], x);
                        for_each_out(p, [&](void* base) {
                            if (p.out_is_bf16) static_cast<uint16_t*>(base)[index] = float_to_bf16_bits(x);
                            else static_cast<float*>(base)[index] = x;
                        });
                    }
                }
            }
        }
        if (lane == 0) umma::tma_store_wait_all();  // staging buffers are read (and the outputs written) before the CTA leaves
        __syncwarp();
    }

    // ---------------------------------------------------------------------- teardown
    // Neither CTA may leave (or free tensor memory) while the other can still reach its shared or tensor memory.
    umma::tc_fence_before();
    __syncthreads();
    umma::cluster_sync_all();
    if (warp == 1) {
        umma::tc_fence_after();
        umma::tmem_dealloc_pair(tmem_base, T::kAlloc);
    }
}

}  // namespace gemm
}  // namespace eider
