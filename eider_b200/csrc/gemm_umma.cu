// Host side of the tcgen05 GEMMs: TMA descriptor encoding, tile-shape selection at plan creation,
// launches, and the C ABI.  Replaces the reference's cuBLASLt NVFP4 / FP8 plans
// (crates/eider-cuda/src/cublaslt/fp4_tn.rs:264-796, fp8_tn.rs:13-292) and its CUTLASS grouped GEMM
// (crates/eider-cuda/native/cutlass_grouped_gemm.cu) with one hand-written kernel family.
#include "gemm_umma.cuh"
#include "decode_umma.cuh"
#include "decode_fp8_umma.cuh"
#include "gemm_pair_umma.cuh"
#include "gemv_stream.cuh"

#include <atomic>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <vector>

#include "eider_b200.h"

namespace eider {
namespace gemm {
namespace {

using EncodeTiled = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                 const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                 CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The driver entry point is looked up at run time so the library loads on machines without a driver.
EncodeTiled encode_fn() {
    static EncodeTiled fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult res;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &res) == cudaSuccess &&
            res == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiled>(ptr);
    });
    return fn;
}

// 2-D byte matrix [rows][row_bytes] with pitch `pitch_bytes`, box = 128 bytes x box_rows, 128-byte swizzle.
cudaError_t make_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t row_bytes, uint64_t pitch_bytes,
                     uint32_t box_rows) {
    EncodeTiled enc = encode_fn();
    if (!enc) return cudaErrorNotSupported;
    if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || pitch_bytes % 16 != 0) return cudaErrorInvalidValue;
    cuuint64_t dims[2] = {row_bytes, rows};
    cuuint64_t strides[1] = {pitch_bytes};
    cuuint32_t box[2] = {kStageBytesK, box_rows};
    cuuint32_t elem[2] = {1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, elem,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}

// Tensor maps a plan has already encoded, keyed by what went into them: encoding costs a driver call of a microsecond or
// two, which is a visible part of a 9 us decode launch.  A plan is driven by one host thread (the reference's contract),
// so the cache is not locked.
struct MapCache {
    static constexpr int kEntries = 8;
    struct Entry {
        const void* base;
        uint64_t rows, row_bytes, pitch;
        uint32_t box_rows;
        CUtensorMap map;
    };
    Entry entries[kEntries];
    uint32_t next;

    cudaError_t get(const CUtensorMap** out, const void* base, uint64_t rows, uint64_t row_bytes, uint64_t pitch, uint32_t box_rows) {
        for (int i = 0; i < kEntries; ++i) {
            Entry& e = entries[i];
            if (e.base == base && e.rows == rows && e.row_bytes == row_bytes && e.pitch == pitch && e.box_rows == box_rows) {
                *out = &e.map;
                return cudaSuccess;
            }
        }
        Entry& e = entries[next % kEntries];
        e.base = nullptr;
        cudaError_t st = make_map(&e.map, base, rows, row_bytes, pitch, box_rows);
        if (st != cudaSuccess) return st;
        e.base = base;
        e.rows = rows;
        e.row_bytes = row_bytes;
        e.pitch = pitch;
        e.box_rows = box_rows;
        ++next;
        *out = &e.map;
        return cudaSuccess;
    }
};

// Per-device caches: one host process may drive several GPUs, and the shared-memory opt-in, the SM count and the
// cluster occupancy all belong to the device that is current at the call.
constexpr int kMaxDevices = 64;

int current_device() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 0;
    return dev;
}

int sm_count() {
    static std::atomic<int> count[kMaxDevices];
    const int dev = current_device();
    int c = count[dev].load(std::memory_order_relaxed);
    if (c == 0) {
        cudaDeviceGetAttribute(&c, cudaDevAttrMultiProcessorCount, dev);
        if (c <= 0) c = 148;
        count[dev].store(c, std::memory_order_relaxed);
    }
    return c;
}

// cudaFuncAttributeMaxDynamicSharedMemorySize is a per-device attribute: opt in once on every device that launches.
template <typename Kernel>
cudaError_t opt_in_smem(std::atomic<uint8_t> (&done)[kMaxDevices], Kernel kernel, uint32_t bytes) {
    const int dev = current_device();
    if (done[dev].load(std::memory_order_acquire)) return cudaSuccess;
    cudaError_t st = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bytes));
    if (st == cudaSuccess) done[dev].store(1, std::memory_order_release);
    return st;
}

template <int KIND, int BLOCK_N, bool TRANSPOSED, int TERMS, bool GROUPED, int EPI_WARPS = 4>
cudaError_t launch(const CUtensorMap& map_rows, const CUtensorMap& map_cols, const Params& p, uint32_t work_items,
                   cudaStream_t stream) {
    constexpr int kStages = default_stages<KIND, BLOCK_N>();
    constexpr uint32_t kSmem = smem_bytes<KIND, BLOCK_N, kStages>();
    auto kernel = gemm_kernel<KIND, BLOCK_N, kStages, TRANSPOSED, TERMS, GROUPED, EPI_WARPS>;
    static std::atomic<uint8_t> configured[kMaxDevices];
    if (cudaError_t st = opt_in_smem(configured, kernel, kSmem); st != cudaSuccess) return st;
    uint32_t grid = static_cast<uint32_t>(sm_count());
    if (work_items < grid) grid = work_items;
    if (grid == 0) return cudaSuccess;
    // Programmatic dependent launch: this kernel's prologue (barriers, tensor memory, first weight tiles) may overlap the
    // tail of the kernel before it; everything that kernel wrote is read only after griddepcontrol.wait.
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(64 + 32 * EPI_WARPS);
    cfg.dynamicSmemBytes = kSmem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, map_rows, map_cols, p);
}

// bf16 output block [rows][cols] with row pitch ld (elements): box = 64 columns x 32 rows, 128-byte swizzle (what the
// epilogue's staging buffers hold)
cudaError_t make_out_map(CUtensorMap* map, void* base, uint64_t rows, uint64_t cols, uint64_t ld) {
    EncodeTiled enc = encode_fn();
    if (!enc) return cudaErrorNotSupported;
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {ld * 2};
    cuuint32_t box[2] = {64, 32};
    cuuint32_t elem[2] = {1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, base, dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}

// CTA-pair kernel: clusters of two along x, as many pairs as can be co-resident (one CTA per SM).
template <int KIND, uint32_t PAIR_N = kPairN>
cudaError_t launch_pair(const CUtensorMap& map_rows, const CUtensorMap& map_cols, const Params& p, uint32_t pair_items,
                        cudaStream_t stream) {
    using L = PairSmem<KIND, PAIR_N>;
    auto kernel = gemm_pair_kernel<KIND, PAIR_N>;
    static std::atomic<int> max_pairs_of[kMaxDevices];
    const int dev = current_device();
    int max_pairs = max_pairs_of[dev].load(std::memory_order_acquire);
    cudaLaunchConfig_t cfg = {};
    cfg.blockDim = dim3(kNumThreads);
    cfg.dynamicSmemBytes = L::kBytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    if (max_pairs == 0) {
        cudaError_t st = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(L::kBytes));
        if (st != cudaSuccess) return st;
        cfg.gridDim = dim3(static_cast<uint32_t>(sm_count()) & ~1u);
        cfg.numAttrs = 1;
        int clusters = 0;
        st = cudaOccupancyMaxActiveClusters(&clusters, kernel, &cfg);
        if (st != cudaSuccess) return st;
        if (clusters <= 0) return cudaErrorLaunchOutOfResources;
        max_pairs = clusters;
        max_pairs_of[dev].store(clusters, std::memory_order_release);
    }
    uint32_t grid_pairs = static_cast<uint32_t>(max_pairs);
    if (pair_items < grid_pairs) grid_pairs = pair_items;
    if (grid_pairs == 0) return cudaSuccess;
    cfg.gridDim = dim3(grid_pairs * 2);
    cfg.numAttrs = 2;
    return cudaLaunchKernelEx(&cfg, kernel, map_rows, map_cols, p);
}

}  // namespace

// ------------------------------------------------------------------------------------ plans
constexpr uint32_t kPairBlockCode = 512;  // DensePlan::block_n value that selects the CTA-pair kernel
constexpr uint32_t kPairNarrowBlockCode = 384;  // ... and its 256 x 192 form
inline bool is_pair_code(uint32_t block_n) { return block_n == kPairBlockCode || block_n == kPairNarrowBlockCode; }

struct DensePlan {
    int kind;
    uint32_t m, n, k;       // tokens, out features, in features
    uint32_t block_n;       // weight rows per tile
    uint32_t* status;       // device status word
    void* peers[8];         // fused all-gather: this rank's column block inside every rank's output (all null = off)
    uint32_t n_peers;
    uint32_t peer_ld;       // row pitch (elements) of those outputs
    CUtensorMap* peer_maps; // device array of n_peers bf16 tensor maps over the same column blocks (TMA-store epilogue)
    void* multicast;        // the same column block inside an NVLink multicast mapping of every rank's output (null = off)
    MapCache maps_x, maps_w;
    // Row-major split K (few tiles, long K): 0 or 1 = off.  The workspace holds `splits` fp32 copies of the output.
    uint32_t splits;
    float* workspace;
    size_t workspace_elems;
};

enum DecodePath : uint32_t { kDecodeAuto = 0, kDecodeStream = 1, kDecodeFused = 2, kDecodeSplit = 3, kDecodeFusedMany = 4 };

struct DecodePlan {
    int kind;
    uint32_t max_tokens, n, k, terms;
    uint32_t splits;
    float* workspace;
    uint32_t* counters;
    uint32_t* status;
    uint32_t fused_splits, fused_per;  // single-launch path for one or two tokens (0 = not available)
    uint32_t many_splits, many_per, many_ring;  // the same kernel as one work item per CTA, three CTAs per SM (0 = not available)
    // activation expansion buffers (NVFP4 W4A16 path)
    uint8_t* act_packed;
    uint8_t* act_scales;
    float* act_col_scale;
    uint32_t path;  // DecodePath: which kernel family serves one or two tokens
    uint32_t ws_splits;  // K splits the scratch was sized for
    MapCache maps_x, maps_w;
};

// Activation of the decode GEMV in operand form: residual NVFP4 terms of up to eight tokens, written once by the producer
// of x and read by every GEMV that consumes x.
struct DecodeOperand {
    uint32_t max_tokens, k;
    uint32_t tokens, terms, cols;  // set by the last expansion: operand rows = tokens * terms, padded to cols = 16 or 32
    uint8_t* packed;               // [32][k / 2]
    uint8_t* sf;                   // [ceil(k / 64)][cols][16]
    float* col_scale;              // [32]
    CUtensorMap map16, map32;      // tiled views of `packed` with 16- and 32-row boxes
};

struct GroupedPlan {
    uint32_t m, max_n, k, groups;  // reference naming: m = out features per expert, max_n = max tokens per expert
    uint32_t* status;
    MapCache maps_a, maps_w;
    // pointer-table entry point: two host-encoded template maps, per-group maps patched on the device, row offsets
    CUtensorMap* templates;   // [2] device copies: rows of a group (box 128 rows), weights of a group (box = column tile)
    CUtensorMap* group_maps;  // [2 * groups]
    uint32_t* offsets;        // [groups + 1] exclusive scan of the per-group row counts of the last call
    CUtensorMap host_templates[2];
};

namespace {

cudaError_t alloc_status(uint32_t** status) {
    cudaError_t st = cudaMalloc(reinterpret_cast<void**>(status), sizeof(uint32_t));
    if (st != cudaSuccess) return st;
    return cudaMemset(*status, 0, sizeof(uint32_t));
}

bool dense_shape_ok(int kind, uint32_t m, uint32_t n, uint32_t k) {
    if (m == 0 || n == 0 || k == 0) return false;
    if (kind == kNvf4) return k % 32 == 0;  // TMA pitch (K/2 bytes) must be a multiple of 16
    return k % 16 == 0;
}

uint32_t pick_block_n(uint32_t m, uint32_t n, uint32_t sms) {
    // Cost model in MMA-cycles per K step: the slowest SM runs `waves` tiles, and an MMA retires in about 128 cycles at
    // N = 256 but never under about 103 however narrow it is, so narrower tiles only pay when they save a whole wave.
    const uint32_t row_tiles = (m + kTileRows - 1) / kTileRows;
    uint32_t best = 64;
    float best_cost = 1e30f;
    // (ties go to the narrower tile: the same number of waves with more SMs streaming; measured, 128 tokens, K 13824 -> N 5120:
    // 18.6 us with 64-wide, 19.7 us with 128-wide tiles; 384 tokens, K 5120 -> N 27648: 29.8 us with 192-wide, 32.5 us with 256-wide)
    for (uint32_t bn : {256u, 192u, 128u, 64u}) {
        const uint32_t tiles = row_tiles * ((n + bn - 1) / bn);
        // (a 192-wide tile is bound by its loads, not by the 103-cycle floor of its MMA: 25.4 us against 22.2 us for the same
        // outputs per SM on 256 x 192 pair tiles, whose cost below is 107)
        const float cost = static_cast<float>((tiles + sms - 1) / sms) * (bn == 256u ? 128.0f : bn == 192u ? 123.0f : 103.0f);
        if (cost <= best_cost) {
            best_cost = cost;
            best = bn;
        }
    }
    // Two or more row tiles: tiles on CTA pairs (each CTA fills only half of the weight tile, measured about 7 % faster than
    // one-CTA 256-wide tiles).  An odd row-tile count wastes half a pair tile, which only large counts amortise.
    // 256 x 192 pair tiles take 0.81 - 0.95 of a 256 x 256 one (0.9 here) and must promise 2 % to be preferred, so they are
    // chosen where they save a turn of the SM pairs.  Measured with K 13824 -> N 5120 (20 against 27 column tiles for 74
    // pairs): 512 tokens 24.6 -> 22.5 us, 1024 tokens 41.6 -> 36.2 us, 2048 tokens 60.0 -> 57.0 us; N 27648 stays with 256
    // (512 tokens: 33.2 against 35.5 us).
    if (row_tiles >= 2 && (row_tiles % 2 == 0 || row_tiles >= 9)) {
        const uint32_t pairs = sms / 2;
        const uint32_t row_pairs = (row_tiles + 1) / 2;
        const uint32_t waves = (row_pairs * ((n + kPairN - 1) / kPairN) + pairs - 1) / pairs;
        const uint32_t narrow_waves = (row_pairs * ((n + kPairNarrowN - 1) / kPairNarrowN) + pairs - 1) / pairs;
        const float cost = static_cast<float>(waves) * 128.0f * 0.93f;
        const float narrow_cost = static_cast<float>(narrow_waves) * 128.0f * 0.93f * 0.9f;
        if (narrow_cost * 1.02f < cost && narrow_cost <= best_cost) return kPairNarrowBlockCode;
        if (cost <= best_cost) return kPairBlockCode;
    }
    return best;
}

// Row-major split K.  A launch whose tiles fill only part of the device streams each tile's whole K through one SM at that
// SM's load rate; splitting K over the idle SMs shortens that at the price of fp32 partial sums written by the GEMM and read
// by a reduce kernel.  The partial sums cost more than the idle SMs give back as soon as there is more than one row tile
// (measured, K 13824 -> N 5120: 64 tokens 19.2 -> 16.7 us and 128 tokens 19.0 -> 18.2 us with three splits, but 256 tokens
// 20.0 -> 29.8 us with two and 512 tokens 24.7 -> 40.7 us with three), so a plan only chooses a split for a single row tile;
// the count comes from a coarse model (0.6 us per 128-byte K stage and wave, partials written at 10 TB/s and read at 6 TB/s,
// 2 us per extra launch, at least eight stages per split, a predicted gain of 15 %).
uint32_t pick_k_splits(int kind, uint32_t m, uint32_t n, uint32_t k, uint32_t block_n, uint32_t sms) {
    const uint32_t row_tiles = (m + kTileRows - 1) / kTileRows;
    if (row_tiles > 1) return 1;
    const uint32_t stages = ((kind == kNvf4 ? k / 2 : k) + kStageBytesK - 1) / kStageBytesK;
    if (stages < 32) return 1;  // (a short K: the second launch costs what the split saves; the measured gains are at 54 stages)
    const bool pair = is_pair_code(block_n);
    const uint32_t slots = pair ? sms / 2 : sms;
    const uint32_t pair_n = block_n == kPairNarrowBlockCode ? kPairNarrowN : kPairN;
    const uint32_t items = pair ? ((row_tiles + 1) / 2) * ((n + pair_n - 1) / pair_n) : row_tiles * ((n + block_n - 1) / block_n);
    if (slots == 0) return 1;
    const float out_mb = static_cast<float>(m) * static_cast<float>(n) * 4.0f * 1e-6f;
    auto cost = [&](uint32_t s) {
        const uint32_t per = (stages + s - 1) / s;
        float t = static_cast<float>((items * s + slots - 1) / slots) * static_cast<float>(per) * 0.6f;
        if (s > 1) t += s * out_mb / 10.0f + 2.0f + (s * out_mb + 0.5f * out_mb) / 6.0f;
        return t;
    };
    uint32_t best = 1;
    float best_cost = cost(1) * 0.85f;
    for (uint32_t s : {2u, 3u, 4u, 5u, 6u, 8u}) {
        const uint32_t per = (stages + s - 1) / s;
        if (per < 8 || (s - 1) * per >= stages || items * s > slots) continue;  // (and the split items still fit in one wave)
        const float c = cost(s);
        if (c < best_cost) {
            best_cost = c;
            best = s;
        }
    }
    return best;
}

// Sets the plan's split count and makes sure the workspace can hold the partial sums (nothing changes on failure).
cudaError_t set_k_splits(DensePlan& plan, uint32_t splits) {
    const uint32_t stages = ((plan.kind == kNvf4 ? plan.k / 2 : plan.k) + kStageBytesK - 1) / kStageBytesK;
    if (splits == 0 || splits > 16) return cudaErrorInvalidValue;
    if (splits > 1 && (splits - 1) * ((stages + splits - 1) / splits) >= stages) return cudaErrorInvalidValue;  // an empty split
    const size_t need = splits > 1 ? static_cast<size_t>(splits) * plan.m * plan.n : 0;
    if (need > plan.workspace_elems) {
        float* ws = nullptr;
        cudaError_t st = cudaMalloc(reinterpret_cast<void**>(&ws), need * sizeof(float));
        if (st != cudaSuccess) return st;
        cudaFree(plan.workspace);
        plan.workspace = ws;
        plan.workspace_elems = need;
    }
    plan.splits = splits;
    return cudaSuccess;
}

}  // namespace

cudaError_t run_dense(DensePlan& plan, const uint8_t* x_values, const uint8_t* x_scales, const uint8_t* w_values,
                      const uint8_t* w_scales, const void* c, void* d, float alpha, float beta, const float* token_scale,
                      const float* channel_scale, int out_is_bf16, cudaStream_t stream) {
    const bool nv = plan.kind == kNvf4;
    if (!x_values || !w_values || !d || (nv && (!x_scales || !w_scales))) return cudaErrorInvalidValue;
    if (beta != 0.0f && !c) return cudaErrorInvalidValue;
    const uint32_t k_bytes = nv ? plan.k / 2 : plan.k;
    const CUtensorMap *map_rows_p, *map_cols_p;
    cudaError_t st = plan.maps_x.get(&map_rows_p, x_values, plan.m, k_bytes, k_bytes, kTileRows);
    if (st != cudaSuccess) return st;
    // (the CTA-pair kernel loads the weight tile in two 128-row halves)
    st = plan.maps_w.get(&map_cols_p, w_values, plan.n, k_bytes, k_bytes, plan.block_n == kPairBlockCode ? kPairHalfN : plan.block_n == kPairNarrowBlockCode ? kPairNarrowN / 2 : plan.block_n);
    if (st != cudaSuccess) return st;
    const CUtensorMap& map_rows = *map_rows_p;
    const CUtensorMap& map_cols = *map_cols_p;
    Params p{};
    p.rows = plan.m;
    p.cols = plan.n;
    p.k_bytes = k_bytes;
    p.row_tiles = (plan.m + kTileRows - 1) / kTileRows;
    p.col_tiles = (plan.n + plan.block_n - 1) / plan.block_n;
    p.k_stages = (k_bytes + kStageBytesK - 1) / kStageBytesK;
    p.sf_rows = x_scales;
    p.sf_cols = w_scales;
    p.sf_tile_stride = ((plan.k / 16 + 3) / 4 * 4) * 128;
    p.out = d;
    p.c_in = c;
    p.ld_out = plan.n;
    p.out_is_bf16 = out_is_bf16;
    p.alpha = alpha;
    p.beta = beta;
    p.row_scale = token_scale;
    p.col_scale = channel_scale;
    p.out_cols = plan.n;
    p.splits = 1;
    p.status = plan.status;
    if (plan.n_peers > 0) {
        if (beta != 0.0f) return cudaErrorInvalidValue;  // C would have to be read from the gathered layout
        for (uint32_t q = 0; q < plan.n_peers; ++q) p.out_peers[q] = plan.peers[q];
        p.n_peers = plan.n_peers;
        p.out = plan.peers[0];
        p.ld_out = plan.peer_ld;
        // plain bf16 output on the CTA-pair kernel: whole tiles leave through shared memory and TMA stores
        if (plan.peer_maps && out_is_bf16 && !channel_scale && is_pair_code(plan.block_n)) p.out_maps = plan.peer_maps;
        // one multicast store per tile instead of one store per peer
        if (plan.multicast && out_is_bf16 && !channel_scale && is_pair_code(plan.block_n) && plan.n % 8 == 0) {
            p.out_multicast = plan.multicast;
            p.out_maps = nullptr;
        }
    }
    // split K: the GEMM writes unscaled fp32 partial sums, one copy of the output per split, and a dependent launch sums,
    // scales and converts them (not with the fused all-gather, whose tiles leave the GPU from the GEMM's epilogue)
    const bool split = plan.splits > 1 && plan.n_peers == 0;
    SplitRowsReduce red{};
    if (split) {
        red.workspace = plan.workspace;
        red.split_stride = static_cast<size_t>(plan.m) * plan.n;
        red.splits = plan.splits;
        red.rows = plan.m;
        red.cols = plan.n;
        red.ld_out = plan.n;
        red.alpha = alpha;
        red.beta = beta;
        red.row_scale = token_scale;
        red.col_scale = channel_scale;
        red.c_in = c;
        red.out = d;
        red.out_is_bf16 = out_is_bf16;
        p.out = plan.workspace;
        p.c_in = nullptr;
        p.out_is_bf16 = 0;
        p.alpha = 1.0f;
        p.beta = 0.0f;
        p.row_scale = nullptr;
        p.col_scale = nullptr;
        p.splits = plan.splits;
        p.split_stride = red.split_stride;
    }
    auto reduce = [&](cudaError_t launched) {
        if (!split || launched != cudaSuccess) return launched;
        const size_t quads = static_cast<size_t>(plan.m) * ((plan.n + 3) / 4);
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(static_cast<uint32_t>(std::min<size_t>((quads + 255) / 256, static_cast<size_t>(sm_count()) * 8)));
        cfg.blockDim = dim3(256);
        cfg.stream = stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        return cudaLaunchKernelEx(&cfg, splitk_rows_reduce_kernel, red);
    };
    if (plan.block_n == kPairBlockCode) {
        // 256 x 256 tiles on CTA pairs
        p.col_tiles = (plan.n + kPairN - 1) / kPairN;
        const uint32_t pair_items = ((p.row_tiles + 1) / 2) * p.col_tiles * p.splits;
        return reduce(nv ? launch_pair<kNvf4>(map_rows, map_cols, p, pair_items, stream)
                         : launch_pair<kFp8>(map_rows, map_cols, p, pair_items, stream));
    }
    if (plan.block_n == kPairNarrowBlockCode) {
        // 256 x 192 tiles on CTA pairs
        p.col_tiles = (plan.n + kPairNarrowN - 1) / kPairNarrowN;
        const uint32_t pair_items = ((p.row_tiles + 1) / 2) * p.col_tiles * p.splits;
        return reduce(nv ? launch_pair<kNvf4, kPairNarrowN>(map_rows, map_cols, p, pair_items, stream)
                         : launch_pair<kFp8, kPairNarrowN>(map_rows, map_cols, p, pair_items, stream));
    }
    const uint32_t items = p.row_tiles * p.col_tiles * p.splits;
#define EIDER_DENSE(KIND, BN) reduce(launch<KIND, BN, false, 1, false>(map_rows, map_cols, p, items, stream))
    if (nv) {
        if (plan.block_n == 256) return EIDER_DENSE(kNvf4, 256);
        if (plan.block_n == 192) return EIDER_DENSE(kNvf4, 192);
        if (plan.block_n == 128) return EIDER_DENSE(kNvf4, 128);
        return EIDER_DENSE(kNvf4, 64);
    }
    if (plan.block_n == 256) return EIDER_DENSE(kFp8, 256);
    if (plan.block_n == 192) return EIDER_DENSE(kFp8, 192);
    if (plan.block_n == 128) return EIDER_DENSE(kFp8, 128);
    return EIDER_DENSE(kFp8, 64);
#undef EIDER_DENSE
}

// Decode orientation: weights are the row operand (128 output features per tile on the tensor-memory
// lanes), the few tokens (x terms) are the column operand.
cudaError_t run_decode(DecodePlan& plan, uint32_t terms, const uint8_t* x_values, const uint8_t* x_scales,
                       const float* x_col_scale, uint32_t tokens, const uint8_t* w_values, const uint8_t* w_scales, const float* channel_scale,
                       const void* c, void* d, float alpha, float beta, int out_is_bf16, cudaStream_t stream) {
    const bool nv = plan.kind == kNvf4;
    if (!x_values || !w_values || !d || tokens == 0 || tokens > plan.max_tokens) return cudaErrorInvalidValue;
    if (nv && (!x_scales || !w_scales)) return cudaErrorInvalidValue;
    const uint32_t k_bytes = nv ? plan.k / 2 : plan.k;
    const uint32_t cols = tokens * terms;
    uint32_t block_n = 16;
    while (block_n < cols) block_n *= 2;
    if (block_n > 256) return cudaErrorInvalidValue;
    const CUtensorMap *map_rows_p, *map_cols_p;
    cudaError_t st = plan.maps_w.get(&map_rows_p, w_values, plan.n, k_bytes, k_bytes, kTileRows);
    if (st != cudaSuccess) return st;
    st = plan.maps_x.get(&map_cols_p, x_values, cols, k_bytes, k_bytes, block_n);
    if (st != cudaSuccess) return st;
    const CUtensorMap& map_rows = *map_rows_p;
    const CUtensorMap& map_cols = *map_cols_p;
    Params p{};
    p.rows = plan.n;
    p.cols = cols;
    p.k_bytes = k_bytes;
    p.row_tiles = (plan.n + kTileRows - 1) / kTileRows;
    p.col_tiles = 1;
    p.k_stages = (k_bytes + kStageBytesK - 1) / kStageBytesK;
    p.sf_rows = w_scales;
    p.sf_cols = x_scales;
    p.sf_tile_stride = ((plan.k / 16 + 3) / 4 * 4) * 128;
    p.out = d;
    p.c_in = c;
    p.ld_out = plan.n;
    p.out_is_bf16 = out_is_bf16;
    p.alpha = alpha;
    p.beta = beta;
    p.row_scale = channel_scale;
    p.col_scale = x_col_scale;
    p.out_cols = tokens;
    p.splits = plan.splits;
    p.workspace = plan.workspace;
    p.counters = plan.counters;
    p.status = plan.status;
    const uint32_t items = p.row_tiles * p.splits;
    // more than sixteen tokens: the splits' partial sums are added up by a kernel of their own
    p.defer_reduce = (p.splits > 1 && tokens > 16) ? 1u : 0u;
#define EIDER_DECODE(KIND, BN, TERMS) launch<KIND, BN, true, TERMS, false>(map_rows, map_cols, p, items, stream)
    auto dispatch = [&]() -> cudaError_t {
    if (nv) {
        if (terms == 8) {
            switch (block_n) {
                case 16: return EIDER_DECODE(kNvf4, 16, 8);
                case 32: return EIDER_DECODE(kNvf4, 32, 8);
                case 64: return EIDER_DECODE(kNvf4, 64, 8);
                case 128: return EIDER_DECODE(kNvf4, 128, 8);
                default: return EIDER_DECODE(kNvf4, 256, 8);
            }
        }
        if (terms == 4) {
            switch (block_n) {
                case 16: return EIDER_DECODE(kNvf4, 16, 4);
                case 32: return EIDER_DECODE(kNvf4, 32, 4);
                case 64: return EIDER_DECODE(kNvf4, 64, 4);
                case 128: return EIDER_DECODE(kNvf4, 128, 4);
                default: return EIDER_DECODE(kNvf4, 256, 4);
            }
        }
        if (terms == 1) {
            switch (block_n) {
                case 16: return EIDER_DECODE(kNvf4, 16, 1);
                case 32: return EIDER_DECODE(kNvf4, 32, 1);
                case 64: return EIDER_DECODE(kNvf4, 64, 1);
                case 128: return EIDER_DECODE(kNvf4, 128, 1);
                default: return EIDER_DECODE(kNvf4, 256, 1);
            }
        }
        return cudaErrorInvalidValue;
    }
    switch (block_n) {
        case 16: return EIDER_DECODE(kFp8, 16, 1);
        case 32: return EIDER_DECODE(kFp8, 32, 1);
        case 64: return EIDER_DECODE(kFp8, 64, 1);
        case 128: return EIDER_DECODE(kFp8, 128, 1);
        default: return EIDER_DECODE(kFp8, 256, 1);
    }
    };
#undef EIDER_DECODE
    st = dispatch();
    if (st != cudaSuccess || !p.defer_reduce) return st;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((plan.n + 255) / 256, tokens);
    cfg.blockDim = dim3(256);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, splitk_reduce_kernel, p);
}

// Pointer-table form: one warp per group copies the two template maps into shared memory, replaces their addresses with
// the group's table entries (and the row extent with the group's row count, so a row tile that hangs over the end reads
// zeros instead of whatever lies behind the group's buffer) and publishes them; thread 0 of the grid writes the
// exclusive scan of the row counts the GEMM walks.
constexpr uint32_t kMapWarps = 8;
__global__ void __launch_bounds__(kMapWarps * 32) grouped_maps_kernel(const CUtensorMap* __restrict__ templates, CUtensorMap* __restrict__ maps,
                                                                    const uint8_t* const* __restrict__ row_values,
                                                                    const uint8_t* const* __restrict__ col_values,
                                                                    const uint32_t* __restrict__ rows_per_group, uint32_t* __restrict__ offsets,
                                                                    uint32_t groups) {
    __shared__ __align__(128) CUtensorMap staged[kMapWarps][2];
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t g = blockIdx.x * kMapWarps + warp;
    if (blockIdx.x == 0 && threadIdx.x == 0) {
        uint32_t sum = 0;
        for (uint32_t i = 0; i < groups; ++i) {
            offsets[i] = sum;
            sum += rows_per_group[i];
        }
        offsets[groups] = sum;
    }
    if (g >= groups) return;  // (warp-uniform)
    const uint32_t* src = reinterpret_cast<const uint32_t*>(templates);
    uint32_t* dst = reinterpret_cast<uint32_t*>(&staged[warp][0]);
    dst[lane] = src[lane];
    dst[lane + 32] = src[lane + 32];
    __syncwarp();
    if (lane == 0) {
        const uint32_t rows = rows_per_group[g];
        umma::tensormap_replace_address(&staged[warp][0], row_values[g]);
        umma::tensormap_replace_rows(&staged[warp][0], rows ? rows : 1u);
        umma::tensormap_replace_address(&staged[warp][1], col_values[g]);
    }
    __syncwarp();
    umma::tensormap_publish(maps + 2 * g, &staged[warp][0]);
    umma::tensormap_publish(maps + 2 * g + 1, &staged[warp][1]);
}

cudaError_t run_grouped_tables(GroupedPlan& plan, const uint8_t* const* a_values, const uint8_t* const* a_scales,
                               const uint8_t* const* b_values, const uint8_t* const* b_scales, uint16_t* const* output,
                               const float* const* alpha, const uint32_t* tokens_per_expert, cudaStream_t stream) {
    if (!a_values || !a_scales || !b_values || !b_scales || !output || !alpha || !tokens_per_expert || !plan.group_maps)
        return cudaErrorInvalidValue;
    grouped_maps_kernel<<<(plan.groups + kMapWarps - 1) / kMapWarps, kMapWarps * 32, 0, stream>>>(
        plan.templates, plan.group_maps, a_values, b_values, tokens_per_expert, plan.offsets, plan.groups);
    cudaError_t st = cudaGetLastError();
    if (st != cudaSuccess) return st;
    const uint32_t k_bytes = plan.k / 2;
    Params p{};
    p.rows = plan.groups * plan.max_n;
    p.cols = plan.groups * plan.m;
    p.k_bytes = k_bytes;
    p.k_stages = (k_bytes + kStageBytesK - 1) / kStageBytesK;
    p.sf_tile_stride = ((plan.k / 16 + 3) / 4 * 4) * 128;
    p.out = nullptr;
    p.ld_out = plan.m;
    p.out_is_bf16 = 1;
    p.alpha = 1.0f;
    p.out_cols = plan.m;
    p.splits = 1;
    p.group_offsets = plan.offsets;
    p.groups = plan.groups;
    p.group_cols = plan.m;
    p.status = plan.status;
    p.group_maps = plan.group_maps;
    p.tbl_row_scales = a_scales;
    p.tbl_col_scales = b_scales;
    p.tbl_out = output;
    p.tbl_alpha = alpha;
    // upper bound on work items: every group can hold max_n rows
    const uint32_t max_row_tiles = plan.groups * ((plan.max_n + kTileRows - 1) / kTileRows);
    // (the kernel's own map arguments are only prefetched on this path; it loads through the per-group maps)
    if (plan.m % 256 == 0) {
        p.col_tiles = plan.m / 256;
        return launch<kNvf4, 256, false, 1, true>(plan.host_templates[0], plan.host_templates[1], p, max_row_tiles * p.col_tiles, stream);
    }
    p.col_tiles = plan.m / 128;
    return launch<kNvf4, 128, false, 1, true>(plan.host_templates[0], plan.host_templates[1], p, max_row_tiles * p.col_tiles, stream);
}

cudaError_t run_grouped(GroupedPlan& plan, const uint8_t* a_values, const uint8_t* a_scales, const uint8_t* w_values,
                        const uint8_t* w_scales, uint16_t* output, const float* alpha, const uint32_t* expert_offsets,
                        uint32_t total_routes, cudaStream_t stream, uint8_t* act_packed = nullptr, uint8_t* act_scales = nullptr,
                        uint32_t act_tile_bytes = 0) {
    if (!a_values || !a_scales || !w_values || !w_scales || (!output && !act_packed) || !alpha || !expert_offsets || total_routes == 0)
        return cudaErrorInvalidValue;
    const uint32_t k_bytes = plan.k / 2;
    const CUtensorMap *map_rows_p, *map_cols_p;
    cudaError_t st = plan.maps_a.get(&map_rows_p, a_values, total_routes, k_bytes, k_bytes, kTileRows);
    if (st != cudaSuccess) return st;
    st = plan.maps_w.get(&map_cols_p, w_values, static_cast<uint64_t>(plan.groups) * plan.m, k_bytes, k_bytes,
                         plan.m % 256 == 0 ? 256 : 128);
    if (st != cudaSuccess) return st;
    const CUtensorMap& map_rows = *map_rows_p;
    const CUtensorMap& map_cols = *map_cols_p;
    Params p{};
    p.rows = total_routes;
    p.cols = plan.groups * plan.m;
    p.k_bytes = k_bytes;
    p.row_tiles = 0;
    p.k_stages = (k_bytes + kStageBytesK - 1) / kStageBytesK;
    p.sf_rows = a_scales;
    p.sf_cols = w_scales;
    p.sf_tile_stride = ((plan.k / 16 + 3) / 4 * 4) * 128;
    p.out = output;
    p.ld_out = plan.m;
    p.out_is_bf16 = 1;
    p.alpha = 1.0f;
    p.beta = 0.0f;
    p.out_cols = plan.m;
    p.splits = 1;
    p.group_offsets = expert_offsets;
    p.groups = plan.groups;
    p.group_cols = plan.m;
    p.group_alpha = alpha;
    p.status = plan.status;
    p.act_packed = act_packed;
    p.act_scales = act_scales;
    p.act_tile_bytes = act_tile_bytes;
    // upper bound on work items: every expert may add one partial row tile
    const uint32_t max_row_tiles = (total_routes + kTileRows - 1) / kTileRows + plan.groups;
    if (plan.m % 256 == 0) {
        p.col_tiles = plan.m / 256;
        // sixteen epilogue warps: one 64-column step of the SiLU * up quantizer per warp (measured 98 us against 108 us with
        // eight warps on 4096 tokens x top-8, 128 experts, H 2048, I 768)
        if (act_packed) return launch<kNvf4, 256, false, 1, true, 16>(map_rows, map_cols, p, max_row_tiles * p.col_tiles, stream);
        return launch<kNvf4, 256, false, 1, true>(map_rows, map_cols, p, max_row_tiles * p.col_tiles, stream);
    }
    p.col_tiles = plan.m / 128;
    if (act_packed) return launch<kNvf4, 128, false, 1, true, 8>(map_rows, map_cols, p, max_row_tiles * p.col_tiles, stream);
    return launch<kNvf4, 128, false, 1, true>(map_rows, map_cols, p, max_row_tiles * p.col_tiles, stream);
}

}  // namespace gemm
}  // namespace eider

using namespace eider;
using namespace eider::gemm;

extern "C" {

// ---- dense NVFP4 W4A4 GEMM -----------------------------------------------------------------
int eider_b200_nvfp4_gemm_tn_supported(uint32_t m, uint32_t n, uint32_t k) { return dense_shape_ok(kNvf4, m, n, k) ? 1 : 0; }

void* eider_b200_nvfp4_gemm_tn_create(uint32_t m, uint32_t n, uint32_t k) {
    if (!dense_shape_ok(kNvf4, m, n, k)) return nullptr;
    auto* plan = new DensePlan{kNvf4, m, n, k, pick_block_n(m, n, static_cast<uint32_t>(sm_count())), nullptr};
    if (alloc_status(&plan->status) != cudaSuccess) {
        delete plan;
        return nullptr;
    }
    if (set_k_splits(*plan, pick_k_splits(kNvf4, m, n, k, plan->block_n, static_cast<uint32_t>(sm_count()))) != cudaSuccess) plan->splits = 1;  // (no workspace: no split)
    return plan;
}

void eider_b200_nvfp4_gemm_tn_destroy(void* raw) {
    auto* plan = static_cast<DensePlan*>(raw);
    if (!plan) return;
    cudaFree(plan->status);
    cudaFree(plan->peer_maps);
    cudaFree(plan->workspace);
    delete plan;
}

cudaError_t eider_b200_nvfp4_gemm_tn_on_stream(void* raw, const uint8_t* x_values, const uint8_t* x_scales,
                                               const uint8_t* w_values, const uint8_t* w_scales, const void* c, void* d,
                                               float alpha, float beta, const float* token_scale, int out_is_bf16,
                                               cudaStream_t stream) {
    auto* plan = static_cast<DensePlan*>(raw);
    if (!plan || plan->kind != kNvf4) return cudaErrorInvalidValue;
    return run_dense(*plan, x_values, x_scales, w_values, w_scales, c, d, alpha, beta, token_scale, nullptr, out_is_bf16,
                     stream);
}

int eider_b200_gemm_plan_set_block_n(void* raw, uint32_t block_n) {
    auto* plan = static_cast<DensePlan*>(raw);
    if (!plan || (block_n != 64 && block_n != 128 && block_n != 192 && block_n != 256 && !is_pair_code(block_n))) return 0;
    plan->block_n = block_n;
    // the split count goes with the tile shape
    if (set_k_splits(*plan, pick_k_splits(plan->kind, plan->m, plan->n, plan->k, block_n, static_cast<uint32_t>(sm_count()))) != cudaSuccess) plan->splits = 1;
    return 1;
}

cudaError_t eider_b200_gemm_plan_set_k_splits(void* raw, uint32_t splits) {
    auto* plan = static_cast<DensePlan*>(raw);
    if (!plan) return cudaErrorInvalidValue;
    return set_k_splits(*plan, splits);
}

// The plans' own choices as plain functions of the shape and the SM count (no device needed): what a plan created for
// (m, n[, k]) on a device of `sms` SMs starts with.
uint32_t eider_b200_gemm_pick_tile(uint32_t m, uint32_t n, uint32_t sms) {
    if (m == 0 || n == 0 || sms < 2) return 0;
    return pick_block_n(m, n, sms);
}

uint32_t eider_b200_gemm_pick_k_splits(int is_nvfp4, uint32_t m, uint32_t n, uint32_t k, uint32_t block_n, uint32_t sms) {
    if (m == 0 || n == 0 || k == 0 || sms < 2 || block_n == 0) return 0;
    return pick_k_splits(is_nvfp4 ? kNvf4 : kFp8, m, n, k, block_n, sms);
}

uint32_t eider_b200_gemm_plan_k_splits(void* raw) {
    auto* plan = static_cast<DensePlan*>(raw);
    return plan ? (plan->splits > 1 ? plan->splits : 1) : 0;
}

cudaError_t eider_b200_gemm_plan_set_output_peers(void* raw, void* const* peers, uint32_t count, uint32_t ld_out) {
    auto* plan = static_cast<DensePlan*>(raw);
    if (!plan || count > 8 || (count > 0 && (!peers || ld_out < plan->n || ld_out % 16 != 0))) return cudaErrorInvalidValue;
    for (uint32_t q = 0; q < count; ++q)
        if (!peers[q] || (reinterpret_cast<uintptr_t>(peers[q]) & 31) != 0) return cudaErrorInvalidValue;
    // Everything that can fail happens before the plan changes, so a failed call leaves the previous setting in force.
    if (count > 0) {
        CUtensorMap maps[8];
        for (uint32_t q = 0; q < count; ++q) {
            cudaError_t st = make_out_map(&maps[q], peers[q], plan->m, plan->n, ld_out);
            if (st != cudaSuccess) return st;
        }
        CUtensorMap* device_maps = plan->peer_maps;
        if (!device_maps) {
            cudaError_t st = cudaMalloc(reinterpret_cast<void**>(&device_maps), 8 * sizeof(CUtensorMap));
            if (st != cudaSuccess) return st;
        }
        cudaError_t st = cudaMemcpy(device_maps, maps, count * sizeof(CUtensorMap), cudaMemcpyHostToDevice);
        if (st != cudaSuccess) {
            if (!plan->peer_maps) cudaFree(device_maps);
            return st;
        }
        plan->peer_maps = device_maps;
    }
    for (uint32_t q = 0; q < 8; ++q) plan->peers[q] = q < count ? peers[q] : nullptr;
    plan->n_peers = count;
    plan->peer_ld = ld_out;
    return cudaSuccess;
}

cudaError_t eider_b200_gemm_plan_set_output_multicast(void* raw, void* multicast_block) {
    auto* plan = static_cast<DensePlan*>(raw);
    if (!plan || (reinterpret_cast<uintptr_t>(multicast_block) & 15) != 0) return cudaErrorInvalidValue;
    if (multicast_block && plan->n_peers == 0) return cudaErrorInvalidValue;  // the peer list carries the row pitch and is the fallback
    plan->multicast = multicast_block;
    return cudaSuccess;
}

uint32_t eider_b200_gemm_plan_block_n(void* raw) {
    auto* plan = static_cast<DensePlan*>(raw);
    return plan ? plan->block_n : 0;
}

cudaError_t eider_b200_gemm_plan_status(void* raw, uint32_t* host_status) {
    auto* plan = static_cast<DensePlan*>(raw);
    if (!plan || !host_status) return cudaErrorInvalidValue;
    return cudaMemcpy(host_status, plan->status, sizeof(uint32_t), cudaMemcpyDeviceToHost);
}

// ---- dense FP8 E4M3 GEMM ---------------------------------------------------------------------
int eider_b200_fp8_gemm_tn_supported(uint32_t m, uint32_t n, uint32_t k) { return dense_shape_ok(kFp8, m, n, k) ? 1 : 0; }

void* eider_b200_fp8_gemm_tn_create(uint32_t m, uint32_t n, uint32_t k) {
    if (!dense_shape_ok(kFp8, m, n, k)) return nullptr;
    auto* plan = new DensePlan{kFp8, m, n, k, pick_block_n(m, n, static_cast<uint32_t>(sm_count())), nullptr};
    if (alloc_status(&plan->status) != cudaSuccess) {
        delete plan;
        return nullptr;
    }
    if (set_k_splits(*plan, pick_k_splits(kFp8, m, n, k, plan->block_n, static_cast<uint32_t>(sm_count()))) != cudaSuccess) plan->splits = 1;  // (no workspace: no split)
    return plan;
}

void eider_b200_fp8_gemm_tn_destroy(void* raw) { eider_b200_nvfp4_gemm_tn_destroy(raw); }

cudaError_t eider_b200_fp8_gemm_tn_on_stream(void* raw, const uint8_t* x_values, const uint8_t* w_values, const void* c,
                                             void* d, float alpha, float beta, const float* token_scale,
                                             const float* channel_scale, int out_is_bf16, cudaStream_t stream) {
    auto* plan = static_cast<DensePlan*>(raw);
    if (!plan || plan->kind != kFp8) return cudaErrorInvalidValue;
    return run_dense(*plan, x_values, nullptr, w_values, nullptr, c, d, alpha, beta, token_scale, channel_scale,
                     out_is_bf16, stream);
}

// ---- decode (tokens <= 64): weights stream once, tokens ride on the MMA N dimension -----------------
namespace {

uint32_t pick_splits(uint32_t k_stages, uint32_t row_tiles) {
    // Persistent CTAs walk (row tile, K split) items.  Cost model in cycles: a stage of four MMAs retires in about 560
    // cycles whatever its width, and meeting the other splits through global memory costs a few memory round trips per
    // item, so K is only split when the row tiles alone leave most SMs idle.
    const uint32_t sms = static_cast<uint32_t>(sm_count());
    uint32_t best = 1;
    float best_cost = 1e30f;
    for (uint32_t s = 1; s <= k_stages && s <= 32; ++s) {
        const uint32_t per = (k_stages + s - 1) / s;
        if (s > 1 && per * (s - 1) >= k_stages) continue;  // last split would be empty
        const uint32_t rounds = (row_tiles * s + sms - 1) / sms;
        const float cost = static_cast<float>(rounds * per) * 560.0f + (s > 1 ? 6000.0f * rounds : 0.0f);
        if (cost < best_cost) {
            best_cost = cost;
            best = s;
        }
    }
    return best;
}

// K splits of the single-launch decode kernel: every CTA keeps one split for the whole launch and walks row tiles, so
// the cost is (row tiles per CTA group) x (stages per split); at most decode::kMaxLocalStages stages per split.
void pick_fused_splits(uint32_t k_stages, uint32_t row_tiles, uint32_t* splits_out, uint32_t* per_out) {
    const uint32_t sms = static_cast<uint32_t>(sm_count());
    uint32_t best = 0, best_per = 0;
    float best_cost = 1e30f;
    for (uint32_t s = 1; s <= k_stages && s <= 32 && s <= sms; ++s) {
        const uint32_t per = (k_stages + s - 1) / s;
        if (per > decode::kMaxLocalStages || decode::ring_depth(per) < 4) continue;
        if (s > 1 && per * (s - 1) >= k_stages) continue;  // last split would be empty
        const uint32_t groups = sms / s;
        const uint32_t rounds = (row_tiles + groups - 1) / groups;
        // cycles: four MMAs per stage retire in about 560 cycles whatever their width; meeting the other splits in
        // global memory costs a few memory round trips at the end of the launch
        const float cost = static_cast<float>(rounds * per) * 560.0f + (s > 1 ? 5000.0f : 0.0f);
        if (cost < best_cost) {
            best_cost = cost;
            best = s;
            best_per = per;
        }
    }
    *splits_out = best;
    *per_out = best_per;
}

// Shared memory the single-launch decode kernel needs for `ring` weight stages beside `per` resident activation stages.
uint32_t fused_smem_bytes(uint32_t per, uint32_t ring, uint32_t cols = decode::kCols) {
    return decode::kFixedBytes + ring * (decode::kWeightTile + decode::kSfTile) +
           per * (decode::act_tile_bytes(cols) + decode::act_sf_stage_bytes(cols));
}
// The prepared variant keeps the operand stages in the ring.
uint32_t prepared_smem_bytes(uint32_t ring, uint32_t cols) { return fused_smem_bytes(ring, ring, cols); }

// One (row tile, K split) item per CTA with three CTAs resident per SM: splits chosen so that the items just fill
// 3 x SMs slots; every SM then interleaves the MMAs, activation expansion and epilogues of three independent items.
void pick_many_splits(uint32_t k_stages, uint32_t row_tiles, uint32_t* splits_out, uint32_t* per_out, uint32_t* ring_out) {
    *splits_out = *per_out = *ring_out = 0;
    const uint32_t slots = 3 * static_cast<uint32_t>(sm_count());
    uint32_t s = slots / row_tiles;
    if (s < 2) return;
    if (s > 32) s = 32;
    if (s > k_stages) s = k_stages;
    uint32_t per = (k_stages + s - 1) / s;
    s = (k_stages + per - 1) / per;  // no empty split
    if (s < 2 || per > decode::kMaxLocalStages) return;
    uint32_t ring = per < 4 ? per : 4;
    while (ring > 2 && fused_smem_bytes(per, ring) > 74 * 1024) --ring;
    if (fused_smem_bytes(per, ring) > 74 * 1024) return;
    *splits_out = s;
    *per_out = per;
    *ring_out = ring;
}

// FP8 single-launch decode: one (row tile, K split) item per CTA, three CTAs per SM.
void pick_fp8_many_splits(uint32_t k_stages, uint32_t row_tiles, uint32_t* splits_out, uint32_t* per_out, uint32_t* ring_out) {
    *splits_out = *per_out = *ring_out = 0;
    const uint32_t slots = 3 * static_cast<uint32_t>(sm_count());
    uint32_t s = slots / row_tiles;
    if (s < 1) s = 1;
    if (s > 32) s = 32;
    if (s > k_stages) s = k_stages;
    uint32_t per = (k_stages + s - 1) / s;
    if (per > decode_fp8::kMaxPer) return;
    s = (k_stages + per - 1) / per;  // no empty split
    uint32_t ring = per < 4 ? per : 4;
    while (ring > 2 && decode_fp8::smem_bytes(per, ring) > 74 * 1024) --ring;
    if (decode_fp8::smem_bytes(per, ring) > 74 * 1024) return;
    *splits_out = s;
    *per_out = per;
    *ring_out = ring;
}

extern "C++" {
template <typename XT>
cudaError_t launch_fp8_fused_decode(const CUtensorMap& map_w, const decode_fp8::Params& p, cudaStream_t stream) {
    auto kernel = decode_fp8::fp8_decode_fused_kernel<XT>;
    static std::atomic<uint8_t> configured[kMaxDevices];
    if (cudaError_t st = opt_in_smem(configured, kernel, 76 * 1024); st != cudaSuccess) return st;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(p.row_tiles * p.splits);
    cfg.blockDim = dim3(decode_fp8::kThreads);
    cfg.dynamicSmemBytes = decode_fp8::smem_bytes(p.per, p.ring);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, map_w, p);
}
}  // extern "C++"

extern "C++" {
template <int COLS>
cudaError_t launch_fp8_quantized_decode(const CUtensorMap& map_w, const CUtensorMap& map_x, const decode_fp8::Params& p, cudaStream_t stream) {
    auto kernel = decode_fp8::fp8_decode_quantized_kernel<COLS>;
    static std::atomic<uint8_t> configured[kMaxDevices];
    if (cudaError_t st = opt_in_smem(configured, kernel, 76 * 1024); st != cudaSuccess) return st;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(p.row_tiles * p.splits);
    cfg.blockDim = dim3(decode_fp8::kThreads);
    cfg.dynamicSmemBytes = decode_fp8::quantized_smem_bytes(p.ring, COLS);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, map_w, map_x, p);
}
}  // extern "C++"

extern "C++" {
template <int TERMS, typename XT, int COLS = decode::kCols, bool PREPARED = false>
cudaError_t launch_fused_decode(const CUtensorMap& map_w, const decode::Params& p, bool many, cudaStream_t stream,
                                const CUtensorMap* map_x = nullptr) {
    auto kernel = decode::nvfp4_decode_fused_kernel<TERMS, XT, COLS, PREPARED>;
    static std::atomic<uint8_t> configured[kMaxDevices];
    if (cudaError_t st = opt_in_smem(configured, kernel, decode::kSmemBytes); st != cudaSuccess) return st;
    // Programmatic dependent launch: setup and the first weight requests of this kernel overlap the tail of the kernel
    // before it; the kernel waits (griddepcontrol.wait) before it reads x or touches scratch, counters and output.
    cudaLaunchConfig_t cfg = {};
    cfg.blockDim = dim3(64 + p.expand_threads);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (many) {  // one item per CTA, small carve-out so that three CTAs share an SM
        cfg.gridDim = dim3(p.row_tiles * p.splits);
        cfg.dynamicSmemBytes = PREPARED ? prepared_smem_bytes(p.ring, COLS) : fused_smem_bytes(p.per, p.ring, COLS);
    } else {
        cfg.gridDim = dim3((static_cast<uint32_t>(sm_count()) / p.splits) * p.splits);
        cfg.dynamicSmemBytes = decode::kSmemBytes;
    }
    return cudaLaunchKernelEx(&cfg, kernel, map_w, map_x ? *map_x : map_w, p);
}
}  // extern "C++"

DecodePlan* make_decode_plan(int kind, uint32_t max_tokens, uint32_t n, uint32_t k) {
    if (max_tokens == 0 || max_tokens > 64 || n == 0 || k == 0) return nullptr;
    if (kind == kNvf4 && (k % 32 != 0 || k / 8 > 4096)) return nullptr;
    if (kind == kFp8 && k % 16 != 0) return nullptr;
    auto* plan = new DecodePlan{};
    plan->kind = kind;
    plan->max_tokens = max_tokens;
    plan->n = n;
    plan->k = k;
    plan->terms = kind == kNvf4 ? (max_tokens * 8 <= 256 ? 8u : 4u) : 1u;
    const uint32_t k_bytes = kind == kNvf4 ? k / 2 : k;
    const uint32_t row_tiles = (n + kTileRows - 1) / kTileRows;
    plan->splits = pick_splits((k_bytes + kStageBytesK - 1) / kStageBytesK, row_tiles);
    if (kind == kNvf4) pick_fused_splits((k_bytes + kStageBytesK - 1) / kStageBytesK, row_tiles, &plan->fused_splits, &plan->fused_per);
    if (kind == kFp8) pick_fp8_many_splits((k_bytes + kStageBytesK - 1) / kStageBytesK, row_tiles, &plan->many_splits, &plan->many_per, &plan->many_ring);
    if (kind == kNvf4)
        pick_many_splits((k_bytes + kStageBytesK - 1) / kStageBytesK, row_tiles, &plan->many_splits, &plan->many_per, &plan->many_ring);
    uint32_t ws_splits = plan->splits > plan->fused_splits ? plan->splits : plan->fused_splits;
    if (plan->many_splits > ws_splits) ws_splits = plan->many_splits;
    if (kind == kNvf4 && ws_splits < (k_bytes + kStageBytesK - 1) / kStageBytesK / decode::kMaxLocalStages + 1)
        ws_splits = (k_bytes + kStageBytesK - 1) / kStageBytesK / decode::kMaxLocalStages + 1;
    plan->ws_splits = ws_splits;
    const size_t ws = static_cast<size_t>(ws_splits) * row_tiles * kTileRows * max_tokens * sizeof(float);
    const uint32_t rows = max_tokens * plan->terms;
    bool ok = cudaMalloc(reinterpret_cast<void**>(&plan->workspace), ws) == cudaSuccess &&
              cudaMalloc(reinterpret_cast<void**>(&plan->counters), row_tiles * sizeof(uint32_t)) == cudaSuccess &&
              cudaMemset(plan->counters, 0, row_tiles * sizeof(uint32_t)) == cudaSuccess &&
              alloc_status(&plan->status) == cudaSuccess;
    if (ok && kind == kNvf4) {
        const size_t sf = scale_layout_len(rows, k);
        ok = cudaMalloc(reinterpret_cast<void**>(&plan->act_packed), static_cast<size_t>(rows) * (k / 2)) == cudaSuccess &&
             cudaMalloc(reinterpret_cast<void**>(&plan->act_scales), sf) == cudaSuccess &&
             cudaMemset(plan->act_scales, 0, sf) == cudaSuccess &&
             cudaMalloc(reinterpret_cast<void**>(&plan->act_col_scale), rows * sizeof(float)) == cudaSuccess;
    } else if (ok) {
        ok = cudaMalloc(reinterpret_cast<void**>(&plan->act_packed), static_cast<size_t>(max_tokens) * k) == cudaSuccess &&
             cudaMalloc(reinterpret_cast<void**>(&plan->act_col_scale), max_tokens * sizeof(float)) == cudaSuccess;
    }
    if (!ok) {
        cudaFree(plan->workspace); cudaFree(plan->counters); cudaFree(plan->status);
        cudaFree(plan->act_packed); cudaFree(plan->act_scales); cudaFree(plan->act_col_scale);
        delete plan;
        return nullptr;
    }
    return plan;
}

}  // namespace

/* NVFP4 W4A16 decode: y[t][n] = weight_scale_2 * sum_k x[t][k] * e2m1(W[n][k]) * ue4m3(S[n][k/16]) */
void* eider_b200_nvfp4_decode_create(uint32_t max_tokens, uint32_t out_features, uint32_t in_features) {
    return make_decode_plan(kNvf4, max_tokens, out_features, in_features);
}

void* eider_b200_fp8_decode_create(uint32_t max_tokens, uint32_t out_features, uint32_t in_features) {
    return make_decode_plan(kFp8, max_tokens, out_features, in_features);
}

void eider_b200_decode_destroy(void* raw) {
    auto* plan = static_cast<DecodePlan*>(raw);
    if (!plan) return;
    cudaFree(plan->workspace); cudaFree(plan->counters); cudaFree(plan->status);
    cudaFree(plan->act_packed); cudaFree(plan->act_scales); cudaFree(plan->act_col_scale);
    delete plan;
}

int eider_b200_decode_plan_set_path(void* raw, uint32_t path) {
    auto* plan = static_cast<DecodePlan*>(raw);
    if (!plan || path > kDecodeFusedMany) return 0;
    plan->path = path;
    return 1;
}

cudaError_t eider_b200_decode_plan_status(void* raw, uint32_t* host_status) {
    auto* plan = static_cast<DecodePlan*>(raw);
    if (!plan || !host_status) return cudaErrorInvalidValue;
    return cudaMemcpy(host_status, plan->status, sizeof(uint32_t), cudaMemcpyDeviceToHost);
}

cudaError_t eider_b200_nvfp4_w4a16_gemv_on_stream(void* raw, const void* input, int input_is_bf16, uint32_t tokens,
                                                  const uint8_t* w_values, const uint8_t* w_scales_tiled,
                                                  float weight_scale_2, const void* c, void* d, float beta,
                                                  int out_is_bf16, cudaStream_t stream) {
    auto* plan = static_cast<DecodePlan*>(raw);
    if (!plan || plan->kind != kNvf4 || !input || !w_values || !w_scales_tiled || !d || tokens == 0 ||
        tokens > plan->max_tokens)
        return cudaErrorInvalidValue;
    if (beta != 0.0f && !c) return cudaErrorInvalidValue;
    if (tokens <= 2 && plan->path == kDecodeStream) {
        // one or two tokens: CUDA-core streaming GEMV (weights read once at HBM speed, exact products)
        gemv_stream::Params g{};
        g.x = input;
        g.tokens = tokens;
        g.n = plan->n;
        g.k = plan->k;
        g.w = w_values;
        g.sf = w_scales_tiled;
        g.sf_tile_stride = ((plan->k / 16 + 3) / 4 * 4) * 128;
        g.out = d;
        g.c_in = c;
        g.ld_out = plan->n;
        g.out_is_bf16 = out_is_bf16;
        g.alpha = weight_scale_2;
        g.beta = beta;
        if (gemv_stream::supported(g)) return gemv_stream::launch(g, input_is_bf16, stream);
        if (plan->path == kDecodeStream) return cudaErrorInvalidValue;
    }
    const bool many = plan->many_splits != 0 && (plan->path == kDecodeFusedMany || plan->path == kDecodeAuto);
    // the single-launch kernel holds 16 operand rows: up to four bf16 tokens (four terms each) or two f32 tokens (eight
    // terms); every CTA expands its slice token after token, which is worth it up to three tokens (13.7 us against
    // 15.5 us for the expansion kernel + GEMV at K = 5120, N = 13824)
    const uint32_t fused_tokens = input_is_bf16 ? 3u : 2u;
    if (tokens <= fused_tokens && plan->path != kDecodeSplit && (many || plan->fused_splits != 0) && (reinterpret_cast<uintptr_t>(input) & 15) == 0) {
        // one launch: the activation is expanded inside the GEMV CTAs
        const CUtensorMap* map_w_p;
        cudaError_t fst = plan->maps_w.get(&map_w_p, w_values, plan->n, plan->k / 2, plan->k / 2, kTileRows);
        if (fst != cudaSuccess) return fst;
        const CUtensorMap& map_w = *map_w_p;
        decode::Params p{};
        p.x = input;
        p.tokens = tokens;
        p.n = plan->n;
        p.k = plan->k;
        p.k_stages = (plan->k / 2 + kStageBytesK - 1) / kStageBytesK;
        p.splits = many ? plan->many_splits : plan->fused_splits;
        p.per = many ? plan->many_per : plan->fused_per;
        p.ring = many ? plan->many_ring : decode::ring_depth(p.per);
        p.expand_threads = p.per * 32 < 128 ? 128 : p.per * 32;
        p.row_tiles = (plan->n + kTileRows - 1) / kTileRows;
        p.sf_w = w_scales_tiled;
        p.sf_tile_stride = ((plan->k / 16 + 3) / 4 * 4) * 128;
        p.out = d;
        p.c_in = c;
        p.ld_out = plan->n;
        p.out_is_bf16 = out_is_bf16;
        p.alpha = weight_scale_2;
        p.beta = beta;
        p.workspace = plan->workspace;
        p.counters = plan->counters;
        p.status = plan->status;
        if (beta != 0.0f && !c) return cudaErrorInvalidValue;
        // bf16 activations carry 8 mantissa bits: four residual terms already sit below their rounding; f32 gets eight
        return input_is_bf16 ? launch_fused_decode<4, uint16_t>(map_w, p, many, stream) : launch_fused_decode<8, float>(map_w, p, many, stream);
    }
    // bf16 activations carry 8 mantissa bits: four residual terms already sit below their rounding; f32 activations get
    // eight terms whenever the call's tokens fit the 256 operand rows, whatever the plan's capacity is
    const uint32_t terms = input_is_bf16 ? 4u : (tokens * 8 <= plan->max_tokens * plan->terms ? 8u : 4u);
    cudaError_t st = eider_b200_expand_nvfp4_terms_on_stream(input, input_is_bf16, plan->act_packed, plan->act_scales,
                                                             plan->act_col_scale, tokens, plan->k, terms, stream);
    if (st != cudaSuccess) return st;
    return run_decode(*plan, terms, plan->act_packed, plan->act_scales, plan->act_col_scale, tokens, w_values, w_scales_tiled,
                      nullptr, c, d, weight_scale_2, beta, out_is_bf16, stream);
}

void* eider_b200_nvfp4_decode_operand_create(uint32_t max_tokens, uint32_t in_features) {
    if (max_tokens == 0 || max_tokens > 8 || in_features == 0 || in_features % 32 != 0 || in_features / 8 > 4096) return nullptr;
    auto* op = new DecodeOperand{};
    op->max_tokens = max_tokens;
    op->k = in_features;
    const size_t packed_bytes = 32 * static_cast<size_t>(in_features / 2);
    const size_t sf_bytes = static_cast<size_t>((in_features + 63) / 64) * 32 * 16;
    bool ok = cudaMalloc(reinterpret_cast<void**>(&op->packed), packed_bytes) == cudaSuccess &&
              cudaMemset(op->packed, 0, packed_bytes) == cudaSuccess &&
              cudaMalloc(reinterpret_cast<void**>(&op->sf), sf_bytes) == cudaSuccess &&
              cudaMemset(op->sf, 0, sf_bytes) == cudaSuccess &&
              cudaMalloc(reinterpret_cast<void**>(&op->col_scale), 32 * sizeof(float)) == cudaSuccess &&
              cudaMemset(op->col_scale, 0, 32 * sizeof(float)) == cudaSuccess &&
              make_map(&op->map16, op->packed, 16, in_features / 2, in_features / 2, 16) == cudaSuccess &&
              make_map(&op->map32, op->packed, 32, in_features / 2, in_features / 2, 32) == cudaSuccess;
    if (!ok) {
        cudaFree(op->packed); cudaFree(op->sf); cudaFree(op->col_scale);
        delete op;
        return nullptr;
    }
    return op;
}

void eider_b200_nvfp4_decode_operand_destroy(void* raw) {
    auto* op = static_cast<DecodeOperand*>(raw);
    if (!op) return;
    cudaFree(op->packed); cudaFree(op->sf); cudaFree(op->col_scale);
    delete op;
}

cudaError_t eider_b200_nvfp4_decode_operand_expand_on_stream(void* raw, const void* input, int input_is_bf16, uint32_t tokens,
                                                             cudaStream_t stream) {
    auto* op = static_cast<DecodeOperand*>(raw);
    // bf16 activations carry 8 mantissa bits: four residual terms already sit below their rounding; f32 gets eight
    const uint32_t terms = input_is_bf16 ? 4u : 8u;
    if (!op || !input || tokens == 0 || tokens > op->max_tokens || tokens * terms > 32) return cudaErrorInvalidValue;
    op->tokens = tokens;
    op->terms = terms;
    op->cols = tokens * terms <= 16 ? 16u : 32u;
    return expand_nvfp4_terms_launch(input, input_is_bf16, op->packed, op->sf, op->col_scale, tokens, op->k, terms, op->cols, stream);
}

cudaError_t eider_b200_nvfp4_w4a16_gemv_prepared_on_stream(void* raw, const void* operand, const uint8_t* w_values,
                                                           const uint8_t* w_scales_tiled, float weight_scale_2, const void* c,
                                                           void* d, float beta, int out_is_bf16, cudaStream_t stream) {
    auto* plan = static_cast<DecodePlan*>(raw);
    auto* op = static_cast<const DecodeOperand*>(operand);
    if (!plan || plan->kind != kNvf4 || !op || op->tokens == 0 || op->k != plan->k || op->tokens > plan->max_tokens || !w_values ||
        !w_scales_tiled || !d || (beta != 0.0f && !c))
        return cudaErrorInvalidValue;
    const CUtensorMap* map_w_p;
    cudaError_t st = plan->maps_w.get(&map_w_p, w_values, plan->n, plan->k / 2, plan->k / 2, kTileRows);
    if (st != cudaSuccess) return st;
    decode::Params p{};
    p.x_sf = op->sf;
    p.x_col_scale = op->col_scale;
    p.tokens = op->tokens;
    p.n = plan->n;
    p.k = plan->k;
    p.k_stages = (plan->k / 2 + kStageBytesK - 1) / kStageBytesK;
    // one (row tile, K split) item per CTA as in the expanding kernel; shapes too small for that split run unsplit or with
    // just enough splits to keep a CTA's stage count in range (the grid may then take more than one wave)
    p.splits = plan->many_splits ? plan->many_splits : 1;
    p.per = (p.k_stages + p.splits - 1) / p.splits;
    while (p.per > decode::kMaxLocalStages) {
        ++p.splits;
        p.per = (p.k_stages + p.splits - 1) / p.splits;
    }
    p.splits = (p.k_stages + p.per - 1) / p.per;  // no empty split
    if (p.splits > plan->ws_splits) return cudaErrorInvalidValue;
    p.ring = p.per < 4 ? p.per : 4;
    while (p.ring > 2 && prepared_smem_bytes(p.ring, op->cols) > 74 * 1024) --p.ring;
    p.expand_threads = 128;
    p.row_tiles = (plan->n + kTileRows - 1) / kTileRows;
    p.sf_w = w_scales_tiled;
    p.sf_tile_stride = ((plan->k / 16 + 3) / 4 * 4) * 128;
    p.out = d;
    p.c_in = c;
    p.ld_out = plan->n;
    p.out_is_bf16 = out_is_bf16;
    p.alpha = weight_scale_2;
    p.beta = beta;
    p.workspace = plan->workspace;
    p.counters = plan->counters;
    p.status = plan->status;
    if (op->cols == 16)
        return op->terms == 4 ? launch_fused_decode<4, uint16_t, 16, true>(*map_w_p, p, true, stream, &op->map16)
                              : launch_fused_decode<8, uint16_t, 16, true>(*map_w_p, p, true, stream, &op->map16);
    return op->terms == 4 ? launch_fused_decode<4, uint16_t, 32, true>(*map_w_p, p, true, stream, &op->map32)
                          : launch_fused_decode<8, uint16_t, 32, true>(*map_w_p, p, true, stream, &op->map32);
}

/* FP8 W8A8 decode with per-token dynamic activation scales:
 * y[t][n] = (sum_k e4m3(xq[t][k]) * e4m3(w[n][k])) * s_x[t] * s_w[n] */
cudaError_t eider_b200_fp8_linear_decode_on_stream(void* raw, const void* input, int input_is_bf16, uint32_t tokens,
                                                   const uint8_t* weight, const float* channel_scale, float weight_scale,
                                                   void* d, int out_is_bf16, cudaStream_t stream) {
    auto* plan = static_cast<DecodePlan*>(raw);
    if (!plan || plan->kind != kFp8 || !input || !weight || !d || tokens == 0 || tokens > plan->max_tokens)
        return cudaErrorInvalidValue;
    // (every CTA quantizes all tokens: beyond four the quantize kernel + GEMV pair is faster, 19.8 us against 23.9 us at
    // eight tokens, K = 5120, N = 7168)
    if (tokens <= decode_fp8::kMaxTokens && plan->many_splits != 0 && plan->path != kDecodeSplit &&
        (reinterpret_cast<uintptr_t>(input) & 15) == 0 && plan->k % 16 == 0) {
        // one launch: the per-token quantizer runs inside the GEMV CTAs
        const CUtensorMap* map_w_p;
        cudaError_t fst = plan->maps_w.get(&map_w_p, weight, plan->n, plan->k, plan->k, kTileRows);
        if (fst != cudaSuccess) return fst;
        const CUtensorMap& map_w = *map_w_p;
        decode_fp8::Params p{};
        p.x = input;
        p.tokens = tokens;
        p.n = plan->n;
        p.k = plan->k;
        p.k_stages = (plan->k + kStageBytesK - 1) / kStageBytesK;
        p.splits = plan->many_splits;
        p.per = plan->many_per;
        p.ring = plan->many_ring;
        p.row_tiles = (plan->n + kTileRows - 1) / kTileRows;
        p.channel_scale = channel_scale;
        p.out = d;
        p.ld_out = plan->n;
        p.out_is_bf16 = out_is_bf16;
        p.alpha = weight_scale;
        p.workspace = plan->workspace;
        p.counters = plan->counters;
        p.status = plan->status;
        return input_is_bf16 ? launch_fp8_fused_decode<uint16_t>(map_w, p, stream) : launch_fp8_fused_decode<float>(map_w, p, stream);
    }
    cudaError_t st;
    if (input_is_bf16)
        st = eider_b200_quantize_fp8_e4m3_dynamic_bf16_batch_on_stream(static_cast<const uint16_t*>(input), plan->act_packed,
                                                                       plan->act_col_scale, tokens, plan->k, stream);
    else
        st = infer_quantize_fp8_e4m3_dynamic_f32_batch_on_stream(static_cast<const float*>(input), plan->act_packed,
                                                                 plan->act_col_scale, tokens, plan->k, stream);
    if (st != cudaSuccess) return st;
    return eider_b200_fp8_linear_decode_quantized_on_stream(raw, plan->act_packed, plan->act_col_scale, tokens, weight, channel_scale,
                                                            weight_scale, d, out_is_bf16, stream);
}

/* The same linear on activations that are already E4M3 codes with one scale per token (the output of the per-token
 * quantizer, run by the producer of x or by the call above). */
cudaError_t eider_b200_fp8_linear_decode_quantized_on_stream(void* raw, const uint8_t* x_codes, const float* x_scale, uint32_t tokens,
                                                             const uint8_t* weight, const float* channel_scale, float weight_scale,
                                                             void* d, int out_is_bf16, cudaStream_t stream) {
    auto* plan = static_cast<DecodePlan*>(raw);
    if (!plan || plan->kind != kFp8 || !x_codes || !x_scale || !weight || !d || tokens == 0 || tokens > plan->max_tokens)
        return cudaErrorInvalidValue;
    const uint32_t cols = tokens <= 16 ? 16u : tokens <= 32 ? 32u : 64u;
    uint32_t ring = plan->many_per < 4 ? plan->many_per : 4;
    while (ring > 2 && decode_fp8::quantized_smem_bytes(ring, cols) > 74 * 1024) --ring;
    if (plan->many_splits == 0 || plan->path == kDecodeSplit || (reinterpret_cast<uintptr_t>(x_codes) & 15) != 0 || plan->k % 16 != 0 ||
        decode_fp8::quantized_smem_bytes(ring, cols) > 74 * 1024)
        // persistent split-K GEMM kernel in the decode orientation
        return run_decode(*plan, 1, x_codes, nullptr, x_scale, tokens, weight, nullptr, channel_scale, nullptr, d, weight_scale, 0.0f,
                          out_is_bf16, stream);
    const CUtensorMap *map_w_p, *map_x_p;
    cudaError_t st = plan->maps_w.get(&map_w_p, weight, plan->n, plan->k, plan->k, kTileRows);
    if (st != cudaSuccess) return st;
    st = plan->maps_x.get(&map_x_p, x_codes, tokens, plan->k, plan->k, cols);
    if (st != cudaSuccess) return st;
    decode_fp8::Params p{};
    p.tokens = tokens;
    p.n = plan->n;
    p.k = plan->k;
    p.k_stages = (plan->k + kStageBytesK - 1) / kStageBytesK;
    p.splits = plan->many_splits;
    p.per = plan->many_per;
    p.ring = ring;
    p.row_tiles = (plan->n + kTileRows - 1) / kTileRows;
    p.channel_scale = channel_scale;
    p.out = d;
    p.ld_out = plan->n;
    p.out_is_bf16 = out_is_bf16;
    p.alpha = weight_scale;
    p.workspace = plan->workspace;
    p.counters = plan->counters;
    p.status = plan->status;
    p.x_scale = x_scale;
    // more than sixteen tokens: the splits' partial sums are added up by a kernel of their own
    p.defer_reduce = (tokens > 16 && p.splits > 1) ? 1u : 0u;
    if (cols == 16) st = launch_fp8_quantized_decode<16>(*map_w_p, *map_x_p, p, stream);
    else if (cols == 32) st = launch_fp8_quantized_decode<32>(*map_w_p, *map_x_p, p, stream);
    else st = launch_fp8_quantized_decode<64>(*map_w_p, *map_x_p, p, stream);
    if (st != cudaSuccess || !p.defer_reduce) return st;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((plan->n + 255) / 256, tokens);
    cfg.blockDim = dim3(256);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, decode_fp8::splitk_reduce_kernel, p);
}


// ---- stateless entry points of the reference, served by cached plans --------------------------------------------
namespace {

// The reference's GEMV / FP8-linear calls carry no plan.  The kernels here need one (split-K scratch, counters, a status
// word), so these entry points keep one decode plan per (device, kind, out features, in features), created by the first
// call with that shape.  That first call allocates and must therefore come before any stream capture; later calls only
// launch.  Calls with the same shape share the plan's scratch and must not overlap on the GPU.
struct ShimPlans {
    struct Entry {
        int dev, kind;
        uint32_t max_tokens, n, k;
        DecodePlan* plan;
    };
    std::mutex mutex;
    std::vector<Entry> entries;

    DecodePlan* get(int kind, uint32_t max_tokens, uint32_t n, uint32_t k) {
        const int dev = current_device();
        std::lock_guard<std::mutex> lock(mutex);
        for (const Entry& e : entries)
            if (e.dev == dev && e.kind == kind && e.max_tokens >= max_tokens && e.n == n && e.k == k) return e.plan;
        DecodePlan* plan = make_decode_plan(kind, max_tokens, n, k);
        if (plan) entries.push_back({dev, kind, max_tokens, n, k, plan});
        return plan;
    }
};
ShimPlans g_shim_plans;

}  // namespace

/* crates/eider-cuda/src/ffi.rs:576-588 (crates/eider-cuda/native/cutlass_gemv.cu:165-243): W4A4 GEMV, d[m] = alpha *
 * sum_k a[m][k] * b[k]; a = weight rows with tiled scales (outer = output feature), b = one NVFP4 activation row with
 * tiled scales (outer = 0); c must be non-null as in the reference and is not read (its beta is 0). */
int infer_cutlass_fp4_gemv_f32_supported(uint32_t m, uint32_t k) { return (m > 0 && k > 0 && k % 32 == 0 && k <= 32768) ? 1 : 0; }

cudaError_t infer_cutlass_fp4_gemv_f32_on_stream(const uint8_t* a_values, const uint8_t* a_scales, const uint8_t* b_values,
                                                 const uint8_t* b_scales, const float* c, float* d, uint32_t m, uint32_t k,
                                                 float alpha, cudaStream_t stream) {
    if (!a_values || !a_scales || !b_values || !b_scales || !c || !d || !infer_cutlass_fp4_gemv_f32_supported(m, k))
        return cudaErrorInvalidValue;
    DecodePlan* plan = g_shim_plans.get(kNvf4, 1, m, k);
    if (!plan) return cudaErrorMemoryAllocation;
    return run_decode(*plan, 1, b_values, b_scales, nullptr, 1, a_values, a_scales, nullptr, nullptr, d, alpha, 0.0f, 0, stream);
}

/* crates/eider-cuda/src/ffi.rs:3131 (kernels crates/eider-cuda/native/non_gemm.cu:9826-9863, 9952-10011): one token,
 * per-token dynamic E4M3 activation, per-channel weight scales, f32 output [rows]. */
cudaError_t infer_fp8_linear_channel_scaled_dynamic_f32_on_stream(const float* input, const uint8_t* weight,
                                                                  const float* channel_weight_scale, float* output,
                                                                  uint32_t rows, uint32_t cols, cudaStream_t stream) {
    if (!input || !weight || !channel_weight_scale || !output || rows == 0 || cols == 0 || cols % 16 != 0)
        return cudaErrorInvalidValue;
    DecodePlan* plan = g_shim_plans.get(kFp8, 1, rows, cols);
    if (!plan) return cudaErrorMemoryAllocation;
    return eider_b200_fp8_linear_decode_on_stream(plan, input, 0, 1, weight, channel_weight_scale, 1.0f, output, 0, stream);
}

/* crates/eider-cuda/src/ffi.rs:3151: the same operator that also hands back the quantized activation and its scale
 * (`threads` is the reference's launch width and has no meaning here). */
cudaError_t infer_fp8_linear_channel_scaled_dynamic_quantized_f32_configured_on_stream(
    const float* input, uint8_t* quantized_input, const uint8_t* weight, const float* channel_weight_scale, float* input_scale,
    float* output, uint32_t rows, uint32_t cols, uint32_t threads, cudaStream_t stream) {
    (void)threads;
    if (!input || !quantized_input || !weight || !channel_weight_scale || !input_scale || !output || rows == 0 || cols == 0 ||
        cols % 16 != 0)
        return cudaErrorInvalidValue;
    DecodePlan* plan = g_shim_plans.get(kFp8, 1, rows, cols);
    if (!plan) return cudaErrorMemoryAllocation;
    cudaError_t st = infer_quantize_fp8_e4m3_dynamic_f32_batch_on_stream(input, quantized_input, input_scale, 1, cols, stream);
    if (st != cudaSuccess) return st;
    return run_decode(*plan, 1, quantized_input, nullptr, input_scale, 1, weight, nullptr, channel_weight_scale, nullptr, output,
                      1.0f, 0.0f, 0, stream);
}

/* crates/eider-cuda/src/ffi.rs:3239: static activation scale, per-tensor weight scale:
 * y[n] = (sum_k e4m3(x / input_scale) * e4m3(w[n][k])) * weight_scale * input_scale. */
cudaError_t infer_fp8_linear_w8a8_f32_on_stream(const float* input, const uint8_t* weight, float* output, uint32_t rows,
                                                uint32_t cols, float weight_scale, float input_scale, cudaStream_t stream) {
    if (!input || !weight || !output || rows == 0 || cols == 0 || cols % 16 != 0 || !(input_scale > 0.0f) || !isfinite(input_scale))
        return cudaErrorInvalidValue;
    DecodePlan* plan = g_shim_plans.get(kFp8, 1, rows, cols);
    if (!plan) return cudaErrorMemoryAllocation;
    cudaError_t st = infer_quantize_fp8_e4m3_f32_on_stream(input, plan->act_packed, cols, input_scale, stream);
    if (st != cudaSuccess) return st;
    return run_decode(*plan, 1, plan->act_packed, nullptr, nullptr, 1, weight, nullptr, nullptr, nullptr, output,
                      weight_scale * input_scale, 0.0f, 0, stream);
}

// ---- routed-MoE grouped GEMM --------------------------------------------------------------------------
/* Supersedes infer_cutlass_fp4_grouped_gemm_{supported,create,destroy,on_stream} (crates/eider-cuda/src/ffi.rs:643-667,
 * crates/eider-cuda/native/cutlass_grouped_gemm.cu).  m = out features per expert, max_n = most rows one expert may get,
 * k = in features.  Instead of device pointer tables the kernel takes the base pointers and the expert offsets the
 * tables were derived from (infer_moe_grouped_pointer_tables_on_stream computes exactly base + offset), so the TMA
 * descriptors can be built on the host and nothing is read back. */
int eider_b200_nvfp4_grouped_gemm_supported(uint32_t m, uint32_t max_n, uint32_t k, uint32_t groups) {
    return (m > 0 && max_n > 0 && k > 0 && groups > 0 && m % 128 == 0 && k % 64 == 0) ? 1 : 0;
}

void* eider_b200_nvfp4_grouped_gemm_create(uint32_t m, uint32_t max_n, uint32_t k, uint32_t groups) {
    if (!eider_b200_nvfp4_grouped_gemm_supported(m, max_n, k, groups)) return nullptr;
    auto* plan = new GroupedPlan{m, max_n, k, groups, nullptr, {}, {}, nullptr, nullptr, nullptr, {}};
    if (alloc_status(&plan->status) != cudaSuccess) {
        delete plan;
        return nullptr;
    }
    return plan;
}

/* crates/eider-cuda/src/ffi.rs:643-667: the reference's grouped GEMM over device pointer tables.  The plan additionally owns
 * the per-group tensor maps that a small kernel patches from the tables in front of every GEMM. */
int infer_cutlass_fp4_grouped_gemm_supported(uint32_t m, uint32_t max_n, uint32_t k, uint32_t groups) {
    return (eider_b200_nvfp4_grouped_gemm_supported(m, max_n, k, groups) && groups <= 4096) ? 1 : 0;
}

void* infer_cutlass_fp4_grouped_gemm_create(uint32_t m, uint32_t max_n, uint32_t k, uint32_t groups) {
    if (!infer_cutlass_fp4_grouped_gemm_supported(m, max_n, k, groups)) return nullptr;
    auto* plan = static_cast<GroupedPlan*>(eider_b200_nvfp4_grouped_gemm_create(m, max_n, k, groups));
    if (!plan) return nullptr;
    CUtensorMap* host_templates = plan->host_templates;
    bool ok = cudaMalloc(reinterpret_cast<void**>(&plan->group_maps), 2 * static_cast<size_t>(groups) * sizeof(CUtensorMap)) == cudaSuccess &&
              cudaMemset(plan->group_maps, 0, 2 * static_cast<size_t>(groups) * sizeof(CUtensorMap)) == cudaSuccess &&
              cudaMalloc(reinterpret_cast<void**>(&plan->templates), 2 * sizeof(CUtensorMap)) == cudaSuccess &&
              cudaMalloc(reinterpret_cast<void**>(&plan->offsets), (static_cast<size_t>(groups) + 1) * sizeof(uint32_t)) == cudaSuccess &&
              // (any mapped, 16-byte aligned address encodes; every use replaces it)
              make_map(&host_templates[0], plan->group_maps, max_n, k / 2, k / 2, kTileRows) == cudaSuccess &&
              make_map(&host_templates[1], plan->group_maps, m, k / 2, k / 2, m % 256 == 0 ? 256 : 128) == cudaSuccess &&
              cudaMemcpy(plan->templates, host_templates, 2 * sizeof(CUtensorMap), cudaMemcpyHostToDevice) == cudaSuccess;
    if (!ok) {
        eider_b200_nvfp4_grouped_gemm_destroy(plan);
        return nullptr;
    }
    return plan;
}

void infer_cutlass_fp4_grouped_gemm_destroy(void* plan) { eider_b200_nvfp4_grouped_gemm_destroy(plan); }

cudaError_t infer_cutlass_fp4_grouped_gemm_on_stream(void* raw, const uint8_t* const* a_values, const uint8_t* const* a_scales,
                                                     const uint8_t* const* b_values, const uint8_t* const* b_scales,
                                                     uint16_t* const* output, float* const* alpha, const uint32_t* tokens_per_expert,
                                                     cudaStream_t stream) {
    auto* plan = static_cast<GroupedPlan*>(raw);
    if (!plan) return cudaErrorInvalidValue;
    return run_grouped_tables(*plan, a_values, a_scales, b_values, b_scales, output, const_cast<const float* const*>(alpha),
                              tokens_per_expert, stream);
}

void eider_b200_nvfp4_grouped_gemm_destroy(void* raw) {
    auto* plan = static_cast<GroupedPlan*>(raw);
    if (!plan) return;
    cudaFree(plan->status);
    cudaFree(plan->group_maps);
    cudaFree(plan->templates);
    cudaFree(plan->offsets);
    delete plan;
}

cudaError_t eider_b200_nvfp4_grouped_gemm_on_stream(void* raw, const uint8_t* a_values, const uint8_t* a_scales,
                                                    const uint8_t* w_values, const uint8_t* w_scales_tiled, uint16_t* output,
                                                    const float* alpha, const uint32_t* expert_offsets, uint32_t total_routes,
                                                    cudaStream_t stream) {
    auto* plan = static_cast<GroupedPlan*>(raw);
    if (!plan) return cudaErrorInvalidValue;
    return run_grouped(*plan, a_values, a_scales, w_values, w_scales_tiled, output, alpha, expert_offsets, total_routes, stream);
}

cudaError_t eider_b200_nvfp4_grouped_gemm_silu_quantize_on_stream(void* raw, const uint8_t* a_values, const uint8_t* a_scales,
                                                                  const uint8_t* w_values_interleaved,
                                                                  const uint8_t* w_scales_tiled_interleaved, const float* alpha,
                                                                  const uint32_t* expert_offsets, uint32_t total_routes,
                                                                  uint8_t* packed, uint8_t* scales, uint32_t scale_tile_bytes,
                                                                  cudaStream_t stream) {
    auto* plan = static_cast<GroupedPlan*>(raw);
    // m = 2 * intermediate: 32 interleaved weight rows give one 16-feature block, and the 16-byte packed stores of two blocks
    // need whole 64-column steps
    if (!plan || !packed || !scales || scale_tile_bytes == 0 || plan->m % 128 != 0 || (reinterpret_cast<uintptr_t>(packed) & 15) != 0 ||
        (plan->m / 4) % 16 != 0 || (reinterpret_cast<uintptr_t>(scales) & 1) != 0)
        return cudaErrorInvalidValue;
    return run_grouped(*plan, a_values, a_scales, w_values_interleaved, w_scales_tiled_interleaved, nullptr, alpha, expert_offsets,
                       total_routes, stream, packed, scales, scale_tile_bytes);
}

cudaError_t eider_b200_grouped_plan_status(void* raw, uint32_t* host_status) {
    auto* plan = static_cast<GroupedPlan*>(raw);
    if (!plan || !host_status) return cudaErrorInvalidValue;
    return cudaMemcpy(host_status, plan->status, sizeof(uint32_t), cudaMemcpyDeviceToHost);
}

}  // extern "C"
