// tcgen05 GEMM mainloop shared by the dense prefill GEMM, the decode (weights-as-rows) GEMM and the
// grouped MoE GEMM.
//
// One CTA per SM, persistent over output tiles.  Warp roles:
//   warp 0      TMA producer: operand tiles (cp.async.bulk.tensor, 128-byte swizzle) and, for NVFP4,
//               the 512-byte scale tiles (cp.async.bulk) into a STAGES-deep shared-memory ring;
//   warp 1      MMA issuer: one elected lane copies the stage's scale tiles into tensor memory
//               (tcgen05.cp) and issues four tcgen05.mma per stage, accumulating in tensor memory;
//   warps 2..5  epilogue: tcgen05.ld the 128 x BLOCK_N fp32 accumulator, apply alpha / row / column
//               scales (+ beta * C), convert and store.
// Data layout: both operands are K-major byte matrices ([rows][K/2] packed E2M1 or [rows][K] E4M3); a
// stage holds 128 bytes of K per row (256 NVFP4 or 128 FP8 elements = four MMAs).  The "row" operand
// (128 rows per tile) lands on the 128 tensor-memory lanes, the "column" operand (BLOCK_N rows per
// tile) on tensor-memory columns.
#pragma once

#include <cuda.h>

#include "common.cuh"
#include "umma.cuh"

namespace eider {
namespace gemm {

enum Kind { kNvf4 = 0, kFp8 = 1 };

constexpr uint32_t kTileRows = 128;       // MMA M
constexpr uint32_t kStageBytesK = 128;    // bytes of K per row per stage (one swizzle row)
constexpr uint32_t kNumThreads = 192;     // producer warp, MMA warp, four epilogue warps
constexpr uint32_t kScaleTileBytes = 512; // 128 rows x 4 blocks

struct Params {
    // problem
    uint32_t rows;        // extent of the row operand (tensor-memory lanes)
    uint32_t cols;        // extent of the column operand
    uint32_t k_bytes;     // bytes of K per row (K/2 for NVFP4, K for FP8)
    uint32_t row_tiles;   // ceil(rows / 128)
    uint32_t col_tiles;   // ceil(cols / BLOCK_N)
    uint32_t k_stages;    // ceil(k_bytes / 128)
    // NVFP4 block scales in the 128x4 tile layout (null for FP8)
    const uint8_t* sf_rows;
    const uint8_t* sf_cols;
    uint32_t sf_tile_stride;  // bytes between consecutive 128-row scale tiles = padded(K/16) * 128
    // epilogue
    void* out;             // [rows][ld_out] (or [cols][ld_out] when TRANSPOSED)
    const void* c_in;      // optional C with the same layout and dtype as out (beta != 0)
    uint32_t ld_out;
    int out_is_bf16;
    float alpha, beta;
    const float* row_scale;  // per row-operand row, may be null
    const float* col_scale;  // per column-operand row, may be null
    // decode: combine `TERMS` consecutive columns into one output column; split-K
    uint32_t out_cols;       // number of logical output columns (cols / TERMS)
    uint32_t splits;         // K splits (1 = none)
    float* workspace;        // [splits][out_cols][row_tiles*128] fp32 partials
    uint32_t* counters;      // [row_tiles] arrival counters, self-resetting
    uint32_t defer_reduce;   // split K: leave the partial sums in `workspace` for splitk_reduce_kernel (many output columns)
    // Row-major split K (prefill with few tiles and a long K): `out` is an fp32 workspace, split s writes its unscaled
    // partial sums at out + s * split_stride elements, and splitk_rows_reduce_kernel sums, scales and converts them.
    size_t split_stride;     // 0 = not in use
    // grouped (MoE): per-group row ranges of the row operand
    const uint32_t* group_offsets;  // [groups + 1] or null
    uint32_t groups;
    uint32_t group_cols;            // column-operand rows per group (weights per expert)
    const float* group_alpha;       // per-group alpha (null: use alpha)
    uint32_t* status;               // device status word, 0 = ok
    // Fused all-gather (dense, row-major bf16/f32 output only): when n_peers > 0 every output element is written to
    // each of out_peers[0 .. n_peers) instead of `out`; the pointers are this rank's column block inside every rank's
    // full output (peer memory mapped into this process), so the slab travels over NVLink tile by tile while the GEMM
    // is still running.  Plain stores only.
    void* out_peers[8];
    uint32_t n_peers;
    // The same destinations as 2-D bf16 tensor maps in global memory (box 64 columns x 32 rows, 128-byte swizzle),
    // n_peers of them: the CTA-pair kernel stages each warp's 32 x 64 block in shared memory and lets the TMA write
    // whole 128-byte lines, which is what makes stores over NVLink efficient.  Null: plain stores.
    const CUtensorMap* out_maps;
    // The same column block once more, as an address inside an NVLink multicast mapping that covers every rank's output
    // (this rank's included).  When set, the CTA-pair kernel writes each staged tile ONCE with multimem.st and the switch
    // replicates it, so a tile leaves this GPU once instead of once per peer.  Stores only.
    void* out_multicast;
    // Grouped GEMM with the SiLU(gate) * up -> NVFP4 quantizer in its epilogue (the down projection's input, without the
    // bf16 round trip): when act_packed is set, the weight rows of every group are interleaved [16 gate rows, 16 up rows]
    // so that 32 consecutive accumulator columns are one 16-feature block of both halves; the epilogue rounds them to bf16
    // (what the unfused GEMM stores), applies SiLU * up and writes packed codes [route][group_cols / 4] and the scale bytes
    // into the group's 128-row scale tiles.  `out` is not written.
    uint8_t* act_packed;
    uint8_t* act_scales;
    uint32_t act_tile_bytes;
    // Pointer-table form of the grouped GEMM (null: base pointers + offsets).  Every group has its own operand, scale,
    // output and alpha pointers in device arrays; `group_maps` holds per-group tensor maps (rows of group g at [2g], its
    // weights at [2g + 1]) whose addresses a preceding kernel has patched in from the tables.  `out` is null on this path.
    const CUtensorMap* group_maps;
    const uint8_t* const* tbl_row_scales;
    const uint8_t* const* tbl_col_scales;
    uint16_t* const* tbl_out;
    const float* const* tbl_alpha;
};

// Calls f(base) for every output buffer of the launch.
template <typename F> __device__ __forceinline__ void for_each_out(const Params& p, F f) {
    if (p.n_peers == 0) {
        f(p.out);
        return;
    }
    for (uint32_t q = 0; q < p.n_peers; ++q) f(p.out_peers[q]);
}

template <int BLOCK_N> struct SmemLayout {
    static constexpr uint32_t kA = kTileRows * kStageBytesK;                 // 16 KB
    static constexpr uint32_t kB = BLOCK_N * kStageBytesK;
    static constexpr uint32_t kSfA = 4 * kScaleTileBytes;                    // 2 KB
    static constexpr uint32_t kSfB = (BLOCK_N > 128 ? 2 : 1) * 4 * kScaleTileBytes;
    __host__ __device__ static constexpr uint32_t stage_bytes(bool nvf4) { return kA + kB + (nvf4 ? kSfA + kSfB : 0); }
};

template <int KIND, int BLOCK_N> constexpr int default_stages() {
    constexpr uint32_t per = SmemLayout<BLOCK_N>::stage_bytes(KIND == kNvf4);
    constexpr int s = static_cast<int>((220u * 1024u) / per);
    return s > 8 ? 8 : s;
}

template <int KIND, int BLOCK_N, int STAGES> constexpr uint32_t smem_bytes() {
    return SmemLayout<BLOCK_N>::stage_bytes(KIND == kNvf4) * STAGES + 1024 /*alignment slack*/ + 256 /*barriers*/;
}

// Tensor-memory columns: accumulator stages + (NVFP4) one stage of scale columns.
template <int KIND, int BLOCK_N> struct TmemPlan {
    static constexpr uint32_t kSfACols = KIND == kNvf4 ? 16 : 0;                        // 4 MMAs x 4 columns
    static constexpr uint32_t kSfBCols = KIND == kNvf4 ? (BLOCK_N > 128 ? 32 : 16) : 0;
    static constexpr uint32_t kAccStages = (2 * BLOCK_N + kSfACols + kSfBCols <= 512) ? 2 : 1;
    // When two full accumulators do not fit beside the scale columns, two buffers that share their last /
    // first kOverlapCols columns are used: buffer 0 = [0, N), buffer 1 = [N - 64, 2N - 64).  The epilogue
    // drains the shared columns first and hands the tensor memory back early, so the next tile's MMAs (into
    // the other buffer) run while the rest of the tile is still being stored.
    static constexpr uint32_t kOverlapCols = 64;
    static constexpr bool kOverlap = kAccStages == 1 && (2 * BLOCK_N - kOverlapCols + kSfACols + kSfBCols <= 512);
    static constexpr uint32_t kAccStride = kOverlap ? BLOCK_N - kOverlapCols : BLOCK_N;
    static constexpr uint32_t kAccCols = kOverlap ? 2 * BLOCK_N - kOverlapCols : kAccStages * BLOCK_N;
    static constexpr uint32_t kUsed = kAccCols + kSfACols + kSfBCols;
    static constexpr uint32_t kAlloc = kUsed <= 32 ? 32 : kUsed <= 64 ? 64 : kUsed <= 128 ? 128 : kUsed <= 256 ? 256 : 512;
    static constexpr uint32_t kSfAOffset = kAccCols;
    static constexpr uint32_t kSfBOffset = kSfAOffset + kSfACols;
};

struct TileCoord {
    uint32_t row0;        // first row-operand row of the tile
    uint32_t row_end;     // one past the last valid row (group end for grouped GEMM)
    uint32_t col0;        // first column-operand row (already includes the group's weight offset)
    uint32_t out_col0;    // first output column
    uint32_t group;
    uint32_t sf_row_tile; // index of the 128-row scale tile of the row operand
    uint32_t k_stage0, k_stage1;  // stage range handled by this work item
    uint32_t split;
    uint32_t row_tile;    // index used for split-K bookkeeping
    uint32_t group_row0;  // grouped: first row of the tile's group
};

// Grouped schedule: work items are (128-row tile of a group) x column tiles.  Each CTA walks the group
// table; the walk is cheap (<= a few hundred groups) and identical in all three roles.
struct GroupWalker {
    const uint32_t* offsets;
    uint32_t groups, col_tiles;
    uint32_t g = 0, base = 0;  // base = number of work items before group g
    __device__ bool locate(uint32_t item, uint32_t& group, uint32_t& tile_in_group, uint32_t& col_tile) {
        while (g < groups) {
            uint32_t n = offsets[g + 1] - offsets[g];
            uint32_t items = ((n + kTileRows - 1) / kTileRows) * col_tiles;
            if (item < base + items) {
                uint32_t local = item - base;
                group = g;
                col_tile = local % col_tiles;   // column tiles fastest: CTAs side by side share the rows
                tile_in_group = local / col_tiles;
                return true;
            }
            base += items;
            ++g;
        }
        return false;
    }
};

template <int BLOCK_N, int TERMS, bool GROUPED>
__device__ __forceinline__ bool get_tile(const Params& p, uint32_t item, GroupWalker& walker, TileCoord& t) {
    if (GROUPED) {
        uint32_t group, tile_in_group, col_tile;
        if (!walker.locate(item, group, tile_in_group, col_tile)) return false;
        uint32_t g0 = p.group_offsets[group], g1 = p.group_offsets[group + 1];
        t.row0 = g0 + tile_in_group * kTileRows;
        t.row_end = g1;
        t.group_row0 = g0;
        t.col0 = group * p.group_cols + col_tile * BLOCK_N;
        t.out_col0 = col_tile * BLOCK_N;
        t.group = group;
        // per-group scale tiles start at ((offset + 127) / 128 + group) tiles
        t.sf_row_tile = (g0 + kTileRows - 1) / kTileRows + group + tile_in_group;
        t.k_stage0 = 0;
        t.k_stage1 = p.k_stages;
        t.split = 0;
        t.row_tile = 0;
        return true;
    }
    uint32_t total = p.row_tiles * p.col_tiles * p.splits;
    if (item >= total) return false;
    uint32_t row_tile = item % p.row_tiles;  // row tiles fastest: neighbours share the column tile
    uint32_t rest = item / p.row_tiles;
    uint32_t col_tile = rest % p.col_tiles;
    uint32_t split = rest / p.col_tiles;
    t.row0 = row_tile * kTileRows;
    t.row_end = p.rows;
    t.col0 = col_tile * BLOCK_N;
    t.out_col0 = col_tile * (BLOCK_N / TERMS);
    t.group = 0;
    t.sf_row_tile = row_tile;
    uint32_t per = (p.k_stages + p.splits - 1) / p.splits;
    t.k_stage0 = split * per;
    t.k_stage1 = min(p.k_stages, t.k_stage0 + per);
    t.split = split;
    t.row_tile = row_tile;
    return true;
}

template <bool BF16> __device__ __forceinline__ void store_chunk32(void* out, size_t index, const float (&v)[32]);
template <> __device__ __forceinline__ void store_chunk32<true>(void* out, size_t index, const float (&v)[32]) {
    uint16_t* dst = static_cast<uint16_t*>(out) + index;
    uint32_t w[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
        w[i] = *reinterpret_cast<uint32_t*>(&h);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) reinterpret_cast<uint4*>(dst)[i] = make_uint4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]);
}
template <> __device__ __forceinline__ void store_chunk32<false>(void* out, size_t index, const float (&v)[32]) {
    float* dst = static_cast<float*>(out) + index;
#pragma unroll
    for (int i = 0; i < 8; ++i) reinterpret_cast<float4*>(dst)[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
}

// 32 fp32 accumulator columns -> 32 bf16 (scaled), written with two 32-byte stores.  A thread owns one output row, so
// every store instruction of a warp touches 32 different lines; wider stores halve the number of such instructions.
// `col_scale` (may be null) points at the per-column scales of these 64 columns, 16-byte aligned; every lane reads the
// same addresses, so the loads are broadcasts out of L1.
__device__ __forceinline__ void convert_bf16x64_scaled(const uint32_t* raw, float scale, const float* col_scale, uint32_t (&w)[32]) {
    if (col_scale) {
#pragma unroll
        for (int q = 0; q < 16; ++q) {
            const float4 c = __ldg(reinterpret_cast<const float4*>(col_scale) + q);
            __nv_bfloat162 h0 = __floats2bfloat162_rn(__uint_as_float(raw[4 * q]) * scale * c.x, __uint_as_float(raw[4 * q + 1]) * scale * c.y);
            __nv_bfloat162 h1 = __floats2bfloat162_rn(__uint_as_float(raw[4 * q + 2]) * scale * c.z, __uint_as_float(raw[4 * q + 3]) * scale * c.w);
            w[2 * q] = *reinterpret_cast<uint32_t*>(&h0);
            w[2 * q + 1] = *reinterpret_cast<uint32_t*>(&h1);
        }
        return;
    }
#pragma unroll
    for (int i = 0; i < 32; ++i) {
        __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(raw[2 * i]) * scale, __uint_as_float(raw[2 * i + 1]) * scale);
        w[i] = *reinterpret_cast<uint32_t*>(&h);
    }
}
__device__ __forceinline__ void store_bf16x64(uint16_t* dst, const uint32_t (&w)[32]) {
#pragma unroll
    for (int i = 0; i < 4; ++i)
        asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(dst + 16 * i), "r"(w[8 * i]),
                     "r"(w[8 * i + 1]), "r"(w[8 * i + 2]), "r"(w[8 * i + 3]), "r"(w[8 * i + 4]), "r"(w[8 * i + 5]),
                     "r"(w[8 * i + 6]), "r"(w[8 * i + 7])
                     : "memory");
}
// 64 fp32 accumulator columns of one row -> 64 scaled bf16 at element offset `offset` of every output buffer
__device__ __forceinline__ void store_row64_all(const Params& p, size_t offset, const uint32_t* raw, float scale,
                                                const float* col_scale) {
    uint32_t w[32];
    convert_bf16x64_scaled(raw, scale, col_scale, w);
    for_each_out(p, [&](void* base) { store_bf16x64(static_cast<uint16_t*>(base) + offset, w); });
}

// Fused SiLU * up -> NVFP4 epilogue of the grouped gate/up GEMM: 64 accumulator columns of one row = two 16-feature blocks,
// each as [16 gate, 16 up].  Same operations, in the same order, as the stand-alone kernel on the bf16 GEMM output
// (crates/eider-cuda/native/non_gemm.cu:2835-2875), so both paths give the same bytes.
__device__ __forceinline__ void silu_quantize_store64(const Params& p, const TileCoord& t, uint32_t row, uint32_t c, const uint32_t* raw,
                                                      float rs) {
    const uint32_t features = p.group_cols / 2;     // the activation's row length (intermediate size)
    const uint32_t kb0 = (t.out_col0 + c) / 32;      // first of the two blocks
    uint32_t words[4];
    uint32_t scale_pair = 0;
#pragma unroll
    for (int b = 0; b < 2; ++b) {
        float v[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const float g = bf16_bits_to_float(float_to_bf16_bits(__uint_as_float(raw[32 * b + i]) * rs));
            const float u = bf16_bits_to_float(float_to_bf16_bits(__uint_as_float(raw[32 * b + 16 + i]) * rs));
            v[i] = moe_silu_mul(g, u);
        }
        uint2 bytes;
        scale_pair |= static_cast<uint32_t>(quantize_block16(v, 16, &bytes)) << (8 * b);
        words[2 * b] = bytes.x;
        words[2 * b + 1] = bytes.y;
    }
    *reinterpret_cast<uint4*>(p.act_packed + static_cast<size_t>(row) * (features / 2) + kb0 * 8) = make_uint4(words[0], words[1], words[2], words[3]);
    const size_t base = ((static_cast<size_t>(t.group_row0) + 127) / 128 + t.group) * p.act_tile_bytes;
    *reinterpret_cast<uint16_t*>(p.act_scales + base + tiled_scale_offset(row - t.group_row0, kb0, features)) = static_cast<uint16_t>(scale_pair);
}

// KIND: operand format.  BLOCK_N: column-operand rows per tile.  TRANSPOSED: output is
// [col][row] (decode: rows are output features, columns are tokens).  TERMS: consecutive columns that
// are summed (with their column scales) into one output column.  GROUPED: MoE schedule.
// EPI_WARPS: epilogue warps, 4, 8 or 16.  Eight or sixteen (two or four per tensor-memory lane quadrant, each taking its
// share of the 64-column steps) are for the arithmetic-heavy SiLU * up -> NVFP4 epilogue, which four warps cannot finish in
// the time of a mainloop.
template <int KIND, int BLOCK_N, int STAGES, bool TRANSPOSED, int TERMS, bool GROUPED, int EPI_WARPS = 4>
__global__ void __launch_bounds__(64 + 32 * EPI_WARPS, 1)
gemm_kernel(const __grid_constant__ CUtensorMap map_rows, const __grid_constant__ CUtensorMap map_cols, const Params p) {
    using L = SmemLayout<BLOCK_N>;
    using T = TmemPlan<KIND, BLOCK_N>;
    constexpr bool kNv = KIND == kNvf4;
    constexpr uint32_t kStage = L::stage_bytes(kNv);
    constexpr uint32_t kAcc = T::kAccStages;
    static_assert(BLOCK_N == 16 || BLOCK_N == 32 || BLOCK_N == 64 || BLOCK_N == 128 || BLOCK_N == 192 || BLOCK_N == 256, "BLOCK_N");
    static_assert(BLOCK_N % TERMS == 0, "TERMS must divide BLOCK_N");
    static_assert(!(GROUPED && (TRANSPOSED || TERMS != 1)), "grouped GEMM is row-major, one term");

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    uint8_t* smem_a = smem;
    uint8_t* smem_b = smem_a + STAGES * L::kA;
    uint8_t* smem_sfa = smem_b + STAGES * L::kB;
    uint8_t* smem_sfb = smem_sfa + (kNv ? STAGES * L::kSfA : 0);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * kStage);
    uint64_t* full = bars;                    // [STAGES]
    uint64_t* empty = bars + STAGES;          // [STAGES]
    uint64_t* acc_full = bars + 2 * STAGES;   // [kAcc]
    uint64_t* acc_empty = acc_full + kAcc;    // [kAcc]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + kAcc);
    volatile uint32_t* abort_flag = tmem_slot + 1;
    uint32_t* last_flag = tmem_slot + 2;

    const uint32_t warp = threadIdx.x >> 5;
    const uint32_t lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int i = 0; i < STAGES; ++i) {
            umma::mbar_init(&full[i], 1);
            umma::mbar_init(&empty[i], 1);
        }
        for (uint32_t i = 0; i < kAcc; ++i) {
            umma::mbar_init(&acc_full[i], 1);
            umma::mbar_init(&acc_empty[i], EPI_WARPS);  // one arrival per epilogue warp
        }
        *abort_flag = 0;
        *last_flag = 0;
        umma::fence_barrier_init();
        umma::prefetch_tensormap(&map_rows);
        umma::prefetch_tensormap(&map_cols);
    }
    if (warp == 1) {
        umma::tmem_alloc(tmem_slot, T::kAlloc);
        umma::tmem_relinquish();
    }
    umma::tc_fence_before();
    __syncthreads();
    umma::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (GROUPED) umma::griddep_wait();  // the expert offsets come from a preceding kernel
    GroupWalker walker{p.group_offsets, p.groups, p.col_tiles};

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        // (whole warp walks the schedule, one elected lane issues the copies)
        {
            const bool leader = umma::elect_one();
            uint32_t it = 0;
            TileCoord t;
            bool ok = true;
            bool dep_waited = false;
            uint32_t maps_group = 0xffffffffu;  // pointer tables: the group whose tensor maps this thread has acquired
            for (uint32_t item = blockIdx.x; ok && get_tile<BLOCK_N, TERMS, GROUPED>(p, item, walker, t); item += gridDim.x) {
                // scale tiles past the end of the column operand do not exist in memory: their rows are
                // zero-filled by the TMA and their outputs are never stored, so the copy is skipped
                const uint32_t sf_col_tiles = (p.cols + kTileRows - 1) / kTileRows;
                const uint32_t sf_col_tile0 = t.col0 / kTileRows;
                bool second_sf = BLOCK_N > 128 && (sf_col_tile0 + 1 < sf_col_tiles);
                const CUtensorMap* mrow = &map_rows;
                const CUtensorMap* mcol = &map_cols;
                int32_t row_coord = static_cast<int32_t>(t.row0), col_coord = static_cast<int32_t>(t.col0);
                const uint8_t* sf_row_ptr = kNv ? p.sf_rows + static_cast<size_t>(t.sf_row_tile) * p.sf_tile_stride : nullptr;
                const uint8_t* sf_col_ptr = kNv ? p.sf_cols + static_cast<size_t>(sf_col_tile0) * p.sf_tile_stride : nullptr;
                if constexpr (GROUPED) if (p.group_maps) {
                    // pointer tables: the group's own tensors, coordinates relative to them
                    mrow = p.group_maps + 2 * t.group;
                    mcol = mrow + 1;
                    row_coord = static_cast<int32_t>(t.row0 - t.group_row0);
                    col_coord = static_cast<int32_t>(t.out_col0);
                    sf_row_ptr = p.tbl_row_scales[t.group] + static_cast<size_t>((t.row0 - t.group_row0) / kTileRows) * p.sf_tile_stride;
                    sf_col_ptr = p.tbl_col_scales[t.group] + static_cast<size_t>(t.out_col0 / kTileRows) * p.sf_tile_stride;
                    second_sf = BLOCK_N > 128 && (t.out_col0 / kTileRows + 1 < p.group_cols / kTileRows);
                    if (leader && maps_group != t.group) {
                        // the maps were written by another kernel through the tensor-map proxy
                        umma::tensormap_fence_acquire(mrow);
                        umma::tensormap_fence_acquire(mcol);
                        maps_group = t.group;
                    }
                }
                for (uint32_t s = t.k_stage0; s < t.k_stage1; ++s, ++it) {
                    const uint32_t stage = it % STAGES;
                    const uint32_t phase = (it / STAGES) & 1;
                    if (!__all_sync(0xffffffffu, umma::mbar_wait(&empty[stage], phase ^ 1, abort_flag, p.status, umma::kTimeoutEmpty))) { ok = false; break; }
                    if (!leader) continue;
                    const uint32_t kb = min(4u, (p.k_bytes - s * kStageBytesK + 31) / 32);  // MMAs in this stage
                    uint32_t bytes = L::kA + L::kB;
                    if (kNv) bytes += kb * kScaleTileBytes * (2 + (second_sf ? 1 : 0));
                    umma::mbar_arrive_expect_tx(&full[stage], bytes);
                    const size_t k_off = static_cast<size_t>(s) * 4 * kScaleTileBytes;
                    // Weights do not depend on the kernel that ran before this one, activations usually do (the
                    // quantizer): under a programmatic dependent launch the weight side of the first stage is
                    // requested before the dependency is awaited.
                    auto load_rows = [&]() {
                        umma::tma_load_2d(smem_a + stage * L::kA, mrow, &full[stage], static_cast<int32_t>(s * kStageBytesK), row_coord);
                        if (kNv) umma::bulk_load_1d(smem_sfa + stage * L::kSfA, sf_row_ptr + k_off, kb * kScaleTileBytes, &full[stage]);
                    };
                    auto load_cols = [&]() {
                        umma::tma_load_2d(smem_b + stage * L::kB, mcol, &full[stage], static_cast<int32_t>(s * kStageBytesK), col_coord);
                        if (kNv) {
                            umma::bulk_load_1d(smem_sfb + stage * L::kSfB, sf_col_ptr + k_off, kb * kScaleTileBytes, &full[stage]);
                            if (second_sf)
                                umma::bulk_load_1d(smem_sfb + stage * L::kSfB + 4 * kScaleTileBytes, sf_col_ptr + p.sf_tile_stride + k_off,
                                                   kb * kScaleTileBytes, &full[stage]);
                        }
                    };
                    if (TRANSPOSED) load_rows(); else load_cols();
                    if (!dep_waited) {
                        umma::griddep_wait();
                        dep_waited = true;
                    }
                    if (TRANSPOSED) load_cols(); else load_rows();
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        // The whole warp walks the schedule (so loop state stays warp-uniform and lives in uniform registers);
        // one elected lane issues the tcgen05 instructions.
        {
            const bool leader = umma::elect_one();
            constexpr uint32_t idesc = kNv ? umma::idesc_nvf4(BLOCK_N) : umma::idesc_f8(BLOCK_N);
            constexpr uint32_t kSfbStep = BLOCK_N > 128 ? 8 : 4;  // tensor-memory columns of column-operand scales per MMA
            const uint32_t a_lo0 = umma::desc_lo_sw128(umma::smem_u32(smem_a));
            const uint32_t b_lo0 = umma::desc_lo_sw128(umma::smem_u32(smem_b));
            const uint32_t sfa_lo0 = umma::desc_lo_scales(umma::smem_u32(smem_sfa));
            const uint32_t sfb_lo0 = umma::desc_lo_scales(umma::smem_u32(smem_sfb));
            const uint32_t sfa_tmem = tmem_base + T::kSfAOffset;
            const uint32_t tail_kb = ((p.k_bytes - (p.k_stages - 1) * kStageBytesK) + 31) / 32;  // MMAs in the last stage
            uint32_t it = 0, tile_count = 0;
            TileCoord t;
            bool ok = true;
            for (uint32_t item = blockIdx.x; ok && get_tile<BLOCK_N, TERMS, GROUPED>(p, item, walker, t); item += gridDim.x, ++tile_count) {
                const uint32_t acc = tile_count % kAcc;
                const uint32_t acc_phase = (tile_count / kAcc) & 1;
                if (!__all_sync(0xffffffffu, umma::mbar_wait(&acc_empty[acc], acc_phase ^ 1, abort_flag, p.status, umma::kTimeoutTmemEmpty))) { ok = false; break; }
                umma::tc_fence_after();
                const uint32_t d_tmem = tmem_base + (T::kOverlap ? (tile_count & 1) : acc) * T::kAccStride;
                // a column tile that does not start on a 128-row scale tile starts (col0 % 128) / 32 columns into it
                const uint32_t sfb_sub = (BLOCK_N % 128 != 0) ? (t.col0 % kTileRows) / 32 : 0;
                const uint32_t sfb_tmem = tmem_base + T::kSfBOffset;
                for (uint32_t s = t.k_stage0; s < t.k_stage1; ++s, ++it) {
                    const uint32_t stage = it % STAGES;
                    const uint32_t phase = (it / STAGES) & 1;
                    if (!__all_sync(0xffffffffu, umma::mbar_wait(&full[stage], phase, abort_flag, p.status, umma::kTimeoutFull))) { ok = false; break; }
                    umma::tc_fence_after();
                    // descriptors differ from the per-CTA base only in the start-address field (16-byte units)
                    const uint32_t a_lo = a_lo0 + stage * (L::kA >> 4);
                    const uint32_t b_lo = b_lo0 + stage * (L::kB >> 4);
                    const uint32_t sfa_lo = sfa_lo0 + stage * (L::kSfA >> 4);
                    const uint32_t sfb_lo = sfb_lo0 + stage * (L::kSfB >> 4);
                    const uint32_t first = (s > t.k_stage0) ? 1u : 0u;
                    if (!leader) {
                        // nothing to issue
                    } else if (s + 1 < p.k_stages || tail_kb == 4) {
                        if (kNv) {
#pragma unroll
                            for (uint32_t j = 0; j < 4; ++j) {
                                umma::tc_copy_scales(sfa_tmem + j * 4, umma::make_desc(sfa_lo + j * 32, umma::kDescHiScales));
                                umma::tc_copy_scales(sfb_tmem + j * kSfbStep, umma::make_desc(sfb_lo + j * 32, umma::kDescHiScales));
                                if (BLOCK_N > 128)
                                    umma::tc_copy_scales(sfb_tmem + j * kSfbStep + 4,
                                                         umma::make_desc(sfb_lo + (4 + j) * 32, umma::kDescHiScales));
                            }
                        }
#pragma unroll
                        for (uint32_t j = 0; j < 4; ++j) {
                            const uint64_t a_desc = umma::make_desc(a_lo + j * 2, umma::kDescHiSw128);
                            const uint64_t b_desc = umma::make_desc(b_lo + j * 2, umma::kDescHiSw128);
                            if (kNv)
                                umma::mma_nvf4(d_tmem, a_desc, b_desc, idesc, sfa_tmem + j * 4, sfb_tmem + j * kSfbStep + sfb_sub,
                                               j == 0 ? first : 1u);
                            else
                                umma::mma_f8(d_tmem, a_desc, b_desc, idesc, j == 0 ? first : 1u);
                        }
                    } else {  // last stage of a K that is not a multiple of the stage depth
                        for (uint32_t j = 0; j < tail_kb; ++j) {
                            if (kNv) {
                                umma::tc_copy_scales(sfa_tmem + j * 4, umma::make_desc(sfa_lo + j * 32, umma::kDescHiScales));
                                umma::tc_copy_scales(sfb_tmem + j * kSfbStep, umma::make_desc(sfb_lo + j * 32, umma::kDescHiScales));
                                if (BLOCK_N > 128)
                                    umma::tc_copy_scales(sfb_tmem + j * kSfbStep + 4,
                                                         umma::make_desc(sfb_lo + (4 + j) * 32, umma::kDescHiScales));
                            }
                        }
                        for (uint32_t j = 0; j < tail_kb; ++j) {
                            const uint64_t a_desc = umma::make_desc(a_lo + j * 2, umma::kDescHiSw128);
                            const uint64_t b_desc = umma::make_desc(b_lo + j * 2, umma::kDescHiSw128);
                            if (kNv)
                                umma::mma_nvf4(d_tmem, a_desc, b_desc, idesc, sfa_tmem + j * 4, sfb_tmem + j * kSfbStep + sfb_sub,
                                               j == 0 ? first : 1u);
                            else
                                umma::mma_f8(d_tmem, a_desc, b_desc, idesc, j == 0 ? first : 1u);
                        }
                    }
                    if (leader) umma::tc_commit(&empty[stage]);  // frees the stage once these MMAs (and scale copies) retire
                    __syncwarp();
                }
                if (ok && leader) umma::tc_commit(&acc_full[acc]);
                __syncwarp();
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue warps
        const uint32_t quad = warp & 3;  // tensor-memory lane quadrant this warp may read
        const uint32_t half = (warp - 2) >> 2;  // which share of the column steps (always 0 with four epilogue warps)
        umma::griddep_wait();            // scales / C written by the preceding kernel are read below
        uint32_t tile_count = 0;
        TileCoord t;
        bool ok = true;
        for (uint32_t item = blockIdx.x; ok && get_tile<BLOCK_N, TERMS, GROUPED>(p, item, walker, t); item += gridDim.x, ++tile_count) {
            const uint32_t acc = tile_count % kAcc;
            const uint32_t acc_phase = (tile_count / kAcc) & 1;
            const bool empty_tile = t.k_stage0 >= t.k_stage1;  // a K split with no stages contributes zeros
            if (!umma::mbar_wait(&acc_full[acc], acc_phase, abort_flag, p.status, umma::kTimeoutTmemFull)) { ok = false; break; }
            umma::tc_fence_after();
            const uint32_t row = t.row0 + quad * 32 + lane;
            const bool row_ok = row < t.row_end;
            float rs = GROUPED ? (p.group_alpha ? p.group_alpha[t.group] : p.alpha) : p.alpha;
            if (p.row_scale && row_ok) rs *= p.row_scale[row];
            size_t row_elems = static_cast<size_t>(row) * p.ld_out;  // element offset of this thread's output row from `out`
            if (!TRANSPOSED && !GROUPED) row_elems += static_cast<size_t>(t.split) * p.split_stride;
            bool out_aligned32 = (reinterpret_cast<uintptr_t>(p.out) & 31) == 0;
            if constexpr (GROUPED) if (p.group_maps) {
                // pointer tables: the group's own output buffer and alpha; `out` is null, so the offset carries the address
                const uintptr_t base = reinterpret_cast<uintptr_t>(p.tbl_out[t.group]);
                row_elems = base / 2 + static_cast<size_t>(row - t.group_row0) * p.ld_out;
                out_aligned32 = (base & 31) == 0;
                rs = *p.tbl_alpha[t.group];
            }
            const uint32_t buf = T::kOverlap ? (tile_count & 1) : acc;
            const uint32_t taddr = tmem_base + ((quad * 32) << 16) + buf * T::kAccStride;
            // Fast path (warp-uniform test): a full-width bf16 tile with no column scale and no C input.  64 columns
            // per step, the next step's tensor-memory loads in flight while this one is converted and stored.
            constexpr bool kWide = !TRANSPOSED && (BLOCK_N % 64 == 0);
            bool wide = false;
            if constexpr (kWide) {
                const uint32_t ncols = GROUPED ? p.group_cols : p.cols;
                wide = p.out_is_bf16 && (reinterpret_cast<uintptr_t>(p.col_scale) & 15) == 0 && !(p.beta != 0.0f && p.c_in) && !empty_tile &&
                       t.out_col0 + BLOCK_N <= ncols && (p.ld_out % 16) == 0 && out_aligned32;
            }
            if constexpr (GROUPED && kWide) if (p.act_packed) {
                // SiLU * up -> NVFP4 epilogue.  A rolled loop over the 64-column steps: the per-step body (32 activations and
                // two block quantizations) is long, and unrolled copies of it beside the plain store path would not fit the
                // instruction cache these warps have to themselves.  With eight (sixteen) warps each set takes a half (quarter) of the steps.
                constexpr uint32_t kSteps = BLOCK_N / 64;
                constexpr uint32_t kPer = kSteps / (EPI_WARPS / 4);
                static_assert(kSteps % (EPI_WARPS / 4) == 0, "the epilogue warp sets share the 64-column steps evenly");
                const uint32_t begin = half * kPer, end = begin + kPer;
#pragma unroll 1
                for (uint32_t step = begin; step < end; ++step) {
                    const uint32_t c = (T::kOverlap && buf == 0) ? (BLOCK_N - 64 - step * 64) : step * 64;
                    uint32_t raw[64];
                    umma::tmem_load_32x32(taddr + c, *reinterpret_cast<uint32_t(*)[32]>(&raw[0]));
                    umma::tmem_load_32x32(taddr + c + 32, *reinterpret_cast<uint32_t(*)[32]>(&raw[32]));
                    umma::tmem_load_wait();
                    if (T::kOverlap ? (step == begin) : (step + 1 == end)) {
                        // the columns the next tile's MMAs may overwrite (the shared ones are step 0, which the first half
                        // has just read; the second half never touches them) are in registers
                        umma::tc_fence_before();
                        __syncwarp();
                        if (lane == 0) umma::mbar_arrive(&acc_empty[acc]);
                    }
                    if (row_ok && !empty_tile) silu_quantize_store64(p, t, row, c, raw, rs);
                }
                continue;
            }
            if constexpr (EPI_WARPS > 4) if (half != 0) {
                // the second set of warps only works in the fused epilogue above; elsewhere it keeps the barrier count
                umma::tc_fence_before();
                __syncwarp();
                if (lane == 0) umma::mbar_arrive(&acc_empty[acc]);
                continue;
            }
            if constexpr (kWide) if (wide) {
                constexpr uint32_t kSteps = BLOCK_N / 64;
                const size_t row_offset = row_elems + t.out_col0;
                uint32_t raw[2][64];
                auto col_of = [&](uint32_t step) { return (T::kOverlap && buf == 0) ? (BLOCK_N - 64 - step * 64) : step * 64; };
                auto issue = [&](uint32_t step, uint32_t (&r)[64]) {
                    const uint32_t c = col_of(step);
                    umma::tmem_load_32x32(taddr + c, *reinterpret_cast<uint32_t(*)[32]>(&r[0]));
                    umma::tmem_load_32x32(taddr + c + 32, *reinterpret_cast<uint32_t(*)[32]>(&r[32]));
                };
                issue(0, raw[0]);
#pragma unroll
                for (uint32_t step = 0; step < kSteps; ++step) {
                    umma::tmem_load_wait();
                    if (step + 1 < kSteps) issue(step + 1, raw[(step + 1) & 1]);
                    if (T::kOverlap && step == 0) {
                        // the shared columns are in registers: the MMA warp may start the next tile in the other buffer
                        umma::tc_fence_before();
                        __syncwarp();
                        if (lane == 0) umma::mbar_arrive(&acc_empty[acc]);
                    }
                    if (row_ok)
                        store_row64_all(p, row_offset + col_of(step), &raw[step & 1][0], rs,
                                        p.col_scale ? p.col_scale + (GROUPED ? t.group * p.group_cols : 0) + t.out_col0 + col_of(step) : nullptr);
                }
                if (!T::kOverlap) {
                    umma::tmem_load_wait();
                    umma::tc_fence_before();
                    __syncwarp();
                    if (lane == 0) umma::mbar_arrive(&acc_empty[acc]);
                }
                continue;
            }
#pragma unroll 1
            for (uint32_t ci = 0; ci < BLOCK_N; ci += 32) {
                constexpr uint32_t kChunk = BLOCK_N < 32 ? BLOCK_N : 32;
                // overlapping buffers: buffer 0 shares its last columns, buffer 1 its first ones; drain those first
                const uint32_t c = (T::kOverlap && buf == 0) ? (BLOCK_N - 32 - ci) : ci;
                uint32_t raw[32];
                if (empty_tile) {
#pragma unroll
                    for (int i = 0; i < 32; ++i) raw[i] = 0;
                } else if (kChunk == 32) {
                    umma::tmem_load_32x32(taddr + c, raw);
                } else {
                    uint32_t r16[16];
                    umma::tmem_load_32x16(taddr + c, r16);
#pragma unroll
                    for (int i = 0; i < 16; ++i) { raw[i] = r16[i]; raw[i + 16] = 0; }
                }
                umma::tmem_load_wait();
                if (T::kOverlap && ci + 32 == T::kOverlapCols) {
                    // the shared columns are in registers: the MMA warp may start the next tile in the other buffer
                    umma::tc_fence_before();
                    __syncwarp();
                    if (lane == 0) umma::mbar_arrive(&acc_empty[acc]);
                }
                if (!TRANSPOSED) {
                    float v[32];
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        const uint32_t col = t.out_col0 + c + i;
                        float x = __uint_as_float(raw[i]) * rs;
                        if (p.col_scale) x *= (col < (GROUPED ? p.group_cols : p.cols)) ? p.col_scale[(GROUPED ? t.group * p.group_cols : 0) + col] : 0.0f;
                        v[i] = x;
                    }
                    const uint32_t ncols = GROUPED ? p.group_cols : p.cols;
                    const uint32_t col0 = t.out_col0 + c;
                    if (row_ok && col0 < ncols) {
                        const size_t index = row_elems + col0;
                        const bool full_chunk = (col0 + 32 <= ncols) && (kChunk == 32);
                        const bool aligned = p.out_is_bf16 ? ((index % 8) == 0 && (reinterpret_cast<uintptr_t>(p.out) & 15) == 0)
                                                           : ((index % 4) == 0 && (reinterpret_cast<uintptr_t>(p.out) & 15) == 0);
                        if (p.beta != 0.0f && p.c_in) {
#pragma unroll
                            for (int i = 0; i < 32; ++i) {
                                if (col0 + i < ncols && static_cast<uint32_t>(i) < kChunk) {
                                    float cv = p.out_is_bf16 ? bf16_bits_to_float(static_cast<const uint16_t*>(p.c_in)[index + i])
                                                             : static_cast<const float*>(p.c_in)[index + i];
                                    v[i] = fmaf(p.beta, cv, v[i]);
                                }
                            }
                        }
                        for_each_out(p, [&](void* base) {
                            if (full_chunk && aligned) {
                                if (p.out_is_bf16) store_chunk32<true>(base, index, v);
                                else store_chunk32<false>(base, index, v);
                            } else {
#pragma unroll
                                for (int i = 0; i < 32; ++i) {
                                    if (col0 + i < ncols && static_cast<uint32_t>(i) < kChunk) {
                                        if (p.out_is_bf16) static_cast<uint16_t*>(base)[index + i] = float_to_bf16_bits(v[i]);
                                        else static_cast<float*>(base)[index + i] = v[i];
                                    }
                                }
                            }
                        });
                    }
                } else {
                    // rows are output features, groups of TERMS columns are one token
#pragma unroll
                    for (int g = 0; g < 32 / TERMS; ++g) {
                        if (static_cast<uint32_t>(g * TERMS) >= kChunk) break;
                        const uint32_t ocol = t.out_col0 + (c / TERMS) + g;
                        if (ocol >= p.out_cols) break;
                        float sum = 0.0f;
#pragma unroll
                        for (int j = 0; j < TERMS; ++j) {
                            const uint32_t col = t.col0 + c + g * TERMS + j;
                            const float cs = p.col_scale ? p.col_scale[col] : 1.0f;
                            sum = fmaf(__uint_as_float(raw[g * TERMS + j]), cs, sum);
                        }
                        if (p.splits > 1) {
                            p.workspace[(static_cast<size_t>(t.split) * p.out_cols + ocol) * (p.row_tiles * kTileRows) + row] = sum;
                        } else if (row_ok) {
                            const size_t index = static_cast<size_t>(ocol) * p.ld_out + row;
                            float x = sum * rs;
                            if (p.beta != 0.0f && p.c_in)
                                x = fmaf(p.beta, p.out_is_bf16 ? bf16_bits_to_float(static_cast<const uint16_t*>(p.c_in)[index])
                                                               : static_cast<const float*>(p.c_in)[index], x);
                            if (p.out_is_bf16) static_cast<uint16_t*>(p.out)[index] = float_to_bf16_bits(x);
                            else static_cast<float*>(p.out)[index] = x;
                        }
                    }
                }
            }
            // accumulator drained: hand the tensor-memory stage back to the MMA warp
            if (!T::kOverlap) {
                umma::tc_fence_before();
                __syncwarp();
                if (lane == 0) umma::mbar_arrive(&acc_empty[acc]);
            }

            if (TRANSPOSED && p.splits > 1 && !p.defer_reduce) {
                // split-K: the last CTA to finish a row tile sums the partials in split order.
                __threadfence();
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (threadIdx.x == 64) {
                    uint32_t prev = atomicAdd(&p.counters[t.row_tile], 1u);
                    *last_flag = (prev == p.splits - 1) ? 1u : 0u;
                    if (prev == p.splits - 1) p.counters[t.row_tile] = 0;
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (*last_flag) {
                    __threadfence();
                    if (row_ok) {
                        // four output columns at a time: their partials (up to 8 splits each per pass) are all requested
                        // before any is used, so a pass costs one memory round trip; sums run in split order
                        for (uint32_t ocol0 = 0; ocol0 < p.out_cols; ocol0 += 4) {
                            float sum[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                            for (uint32_t s0 = 0; s0 < p.splits; s0 += 8) {
                                float part[4][8];
#pragma unroll
                                for (uint32_t c = 0; c < 4; ++c)
#pragma unroll
                                    for (uint32_t u = 0; u < 8; ++u)
                                        part[c][u] = (s0 + u < p.splits && ocol0 + c < p.out_cols)
                                                         ? __ldcg(&p.workspace[(static_cast<size_t>(s0 + u) * p.out_cols + ocol0 + c) * (p.row_tiles * kTileRows) + row])
                                                         : 0.0f;
#pragma unroll
                                for (uint32_t c = 0; c < 4; ++c)
#pragma unroll
                                    for (uint32_t u = 0; u < 8; ++u) sum[c] += part[c][u];
                            }
#pragma unroll
                            for (uint32_t c = 0; c < 4; ++c) {
                                if (ocol0 + c >= p.out_cols) break;
                                const size_t index = static_cast<size_t>(ocol0 + c) * p.ld_out + row;
                                float x = sum[c] * rs;
                                if (p.beta != 0.0f && p.c_in)
                                    x = fmaf(p.beta, p.out_is_bf16 ? bf16_bits_to_float(static_cast<const uint16_t*>(p.c_in)[index])
                                                                   : static_cast<const float*>(p.c_in)[index], x);
                                if (p.out_is_bf16) static_cast<uint16_t*>(p.out)[index] = float_to_bf16_bits(x);
                                else static_cast<float*>(p.out)[index] = x;
                            }
                        }
                    }
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");
            }
        }
    }

    // ---------------------------------------------------------------------- teardown
    umma::tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        umma::tc_fence_after();
        umma::tmem_dealloc(tmem_base, T::kAlloc);
    }
}

// Row-major split K: out[r][c] = (sum over splits, in split order, of workspace[s][r][c]) * alpha * row_scale[r] * col_scale[c]
// (+ beta * c_in[r][c]), the operations of the GEMM epilogue in the same order.  Four columns per thread; a programmatic
// dependent launch behind the GEMM.
struct SplitRowsReduce {
    const float* workspace;
    size_t split_stride;
    uint32_t splits, rows, cols, ld_out;
    float alpha, beta;
    const float* row_scale;
    const float* col_scale;
    const void* c_in;
    void* out;
    int out_is_bf16;
};
__global__ void __launch_bounds__(256) splitk_rows_reduce_kernel(const SplitRowsReduce a) {
    umma::griddep_wait();
    const uint32_t quads = (a.cols + 3) / 4;
    const size_t total = static_cast<size_t>(a.rows) * quads;
    for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const uint32_t row = static_cast<uint32_t>(i / quads);
        const uint32_t col = static_cast<uint32_t>(i % quads) * 4;
        const size_t src = static_cast<size_t>(row) * a.cols + col;
        const bool whole = col + 4 <= a.cols && (a.cols % 4) == 0;
        float sum[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        for (uint32_t sp = 0; sp < a.splits; ++sp) {
            const float* part = a.workspace + sp * a.split_stride + src;
            if (whole) {
                const float4 v = __ldcg(reinterpret_cast<const float4*>(part));
                sum[0] += v.x; sum[1] += v.y; sum[2] += v.z; sum[3] += v.w;
            } else {
                for (uint32_t j = 0; j < 4 && col + j < a.cols; ++j) sum[j] += __ldcg(part + j);
            }
        }
        float rs = a.alpha;
        if (a.row_scale) rs *= a.row_scale[row];
        for (uint32_t j = 0; j < 4 && col + j < a.cols; ++j) {
            const size_t index = static_cast<size_t>(row) * a.ld_out + col + j;
            float x = sum[j] * rs;
            if (a.col_scale) x *= a.col_scale[col + j];
            if (a.beta != 0.0f && a.c_in)
                x = fmaf(a.beta, a.out_is_bf16 ? bf16_bits_to_float(static_cast<const uint16_t*>(a.c_in)[index])
                                               : static_cast<const float*>(a.c_in)[index], x);
            if (a.out_is_bf16) static_cast<uint16_t*>(a.out)[index] = float_to_bf16_bits(x);
            else static_cast<float*>(a.out)[index] = x;
        }
    }
}

// Sums the K splits' partial sums of the decode orientation when many tokens share the launch: the one CTA per row tile that
// arrives last needs a memory round trip per four tokens, this kernel spreads the same sums (in split order) over the whole
// device.  One thread per (token, output row); a programmatic dependent launch.
__global__ void __launch_bounds__(256) splitk_reduce_kernel(const Params p) {
    umma::griddep_launch_dependents();
    umma::griddep_wait();
    const uint32_t row = blockIdx.x * 256 + threadIdx.x, ocol = blockIdx.y;
    if (row >= p.rows) return;
    const size_t stride = static_cast<size_t>(p.row_tiles) * kTileRows;
    float sum = 0.0f;
    for (uint32_t s0 = 0; s0 < p.splits; s0 += 8) {
        float part[8];
#pragma unroll
        for (uint32_t u = 0; u < 8; ++u)
            part[u] = s0 + u < p.splits ? __ldcg(&p.workspace[(static_cast<size_t>(s0 + u) * p.out_cols + ocol) * stride + row]) : 0.0f;
#pragma unroll
        for (uint32_t u = 0; u < 8; ++u) sum += part[u];
    }
    float x = sum * (p.row_scale ? p.alpha * p.row_scale[row] : p.alpha);
    const size_t index = static_cast<size_t>(ocol) * p.ld_out + row;
    if (p.beta != 0.0f && p.c_in)
        x = fmaf(p.beta, p.out_is_bf16 ? bf16_bits_to_float(static_cast<const uint16_t*>(p.c_in)[index]) : static_cast<const float*>(p.c_in)[index], x);
    if (p.out_is_bf16) static_cast<uint16_t*>(p.out)[index] = float_to_bf16_bits(x);
    else static_cast<float*>(p.out)[index] = x;
}

}  // namespace gemm
}  // namespace eider
