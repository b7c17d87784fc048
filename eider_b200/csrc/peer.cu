// Device-side meeting of the ranks of one node over peer memory (NVLink): a bounded barrier on a small signal pad that
// every rank keeps in memory its peers can write (symmetric memory / CUDA IPC).  The fused all-gather of the dense GEMM
// needs one such meeting per step; the reference is single-GPU and has no counterpart.
//
// Pad layout, per rank: uint32_t flag[channel][source rank] with 8 slots per channel.  Rank r announces epoch e on a
// channel by storing e into flag[channel][r] of every rank's pad (release, system scope) and then waits until all of its
// own flag[channel][*] have reached e (acquire, system scope).  The epoch lives in device memory of the calling rank and
// is advanced by the kernel itself, so a captured graph can be replayed.  Every wait is bounded by a cycle budget; when it
// runs out the kernel records which peer was missing in a status word and returns, leaving the context usable.
#include "common.cuh"
#include "eider_b200.h"

namespace eider {
namespace {

constexpr uint32_t kMaxRanks = 8;
constexpr uint32_t kChannels = 16;

struct PadTable {
    uint32_t* pad[kMaxRanks];
};

__device__ __forceinline__ void store_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t load_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// state[0 .. 16): epoch per channel; state[16]: status (0 = ok, else 0xBA000000 | channel << 8 | missing rank)
__global__ void __launch_bounds__(32) peer_barrier_kernel(PadTable pads, uint32_t world, uint32_t rank, uint32_t channel,
                                                          uint32_t* __restrict__ state, long long timeout_cycles) {
    __shared__ uint32_t epoch_sh;
    if (threadIdx.x == 0) {
        const uint32_t e = state[channel] + 1;
        state[channel] = e;
        epoch_sh = e;
    }
    __syncwarp();
    const uint32_t epoch = epoch_sh;
    const uint32_t q = threadIdx.x;
    if (q >= world) return;
    // everything this rank wrote before the barrier (its GEMM kernel has completed: stream order) is published with the flag
    __threadfence_system();
    store_release_sys(pads.pad[q] + channel * kMaxRanks + rank, epoch);
    const uint32_t* mine = pads.pad[rank] + channel * kMaxRanks + q;
    const long long start = clock64();
    // (epochs are compared as a signed distance so that a wrapped counter still orders correctly)
    while (static_cast<int32_t>(load_acquire_sys(mine) - epoch) < 0) {
        if (clock64() - start > timeout_cycles) {
            atomicCAS(state + kChannels, 0u, 0xBA000000u | (channel << 8) | q);
            return;
        }
        __nanosleep(64);
    }
}


// ---- expert-parallel MoE over peer memory ---------------------------------------------------------------------------
// Experts are split evenly over the ranks (the prescribed partitioning); tokens start sharded by rows.  Instead of a
// collective with host-side split sizes, the routes travel by plain peer stores into buffers every rank keeps in
// peer-writable memory, and every count stays on the device:
//   1. each rank sorts its routes by global expert (the library's stable route sort) and publishes its per-expert counts
//      to every rank (ep_publish_counts);                                                          -- barrier --
//   2. from all ranks' counts every rank derives, for each expert, where the owner's rows of that expert start and how
//      many rows of lower source ranks come first (ep_offsets), quantizes each of its tokens once and stores the NVFP4
//      row, its scale bytes (straight into the owner's per-expert scale tiles) and a return address for every route
//      into the owner's receive buffers, already in expert-major order (ep_dispatch_rows);         -- barrier --
//   3. the owner runs the grouped pipeline on what it received and stores each result row back into the source rank's
//      return buffer at the route's own index (ep_return_rows);                                    -- barrier --
//   4. the source combines its routes with their weights.
// A route costs in_features * 9 / 16 bytes on the way out (NVFP4, not bf16) and 2 * out_features on the way back.
struct ByteTable {
    uint8_t* p[kMaxRanks];
};
struct WordTable {
    uint32_t* p[kMaxRanks];
};

// counts_all is [world][experts] on every rank; this rank writes row `rank` everywhere.
__global__ void ep_publish_counts_kernel(const uint32_t* __restrict__ counts, WordTable counts_all, uint32_t world, uint32_t rank,
                                         uint32_t experts) {
    const uint32_t e = blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= experts) return;
    const uint32_t c = counts[e];
    for (uint32_t q = 0; q < world; ++q) counts_all.p[q][static_cast<size_t>(rank) * experts + e] = c;
}

// One CTA.  expert_base[e]: row, inside the owner's receive buffer, where expert e starts (= the owner's local expert
// offset); before_me[e]: rows of expert e that come from lower source ranks; recv_offsets[0 .. per + 1): this rank's own
// local expert offsets; recv_total[0] = rows this rank receives.
__global__ void __launch_bounds__(1024) ep_offsets_kernel(const uint32_t* __restrict__ counts_all, uint32_t world, uint32_t rank,
                                                          uint32_t experts, uint32_t* __restrict__ expert_base,
                                                          uint32_t* __restrict__ before_me, uint32_t* __restrict__ recv_offsets,
                                                          uint32_t* __restrict__ recv_total) {
    __shared__ uint32_t total[1024];
    const uint32_t per = experts / world;
    const uint32_t e = threadIdx.x;
    uint32_t sum = 0, before = 0;
    if (e < experts) {
        for (uint32_t s = 0; s < world; ++s) {
            const uint32_t c = counts_all[static_cast<size_t>(s) * experts + e];
            if (s < rank) before += c;
            sum += c;
        }
    }
    total[e] = sum;
    __syncthreads();
    if (e >= experts) return;
    const uint32_t owner = e / per;
    uint32_t base = 0;
    for (uint32_t j = owner * per; j < e; ++j) base += total[j];
    expert_base[e] = base;
    before_me[e] = before;
    if (owner == rank) {
        recv_offsets[e - owner * per] = base;
        if (e == owner * per + per - 1) {
            recv_offsets[per] = base + sum;
            recv_total[0] = base + sum;
        }
    }
}

// One warp per local sorted route: the token's NVFP4 row and scale bytes go to the owner of the route's expert.
constexpr uint32_t kDispatchWarps = 8;
__global__ void __launch_bounds__(kDispatchWarps * 32) ep_dispatch_rows_kernel(
    const uint8_t* __restrict__ src_packed, const uint8_t* __restrict__ src_scales, const uint32_t* __restrict__ sorted_routes,
    const uint32_t* __restrict__ sorted_experts, const uint32_t* __restrict__ local_offsets, const uint32_t* __restrict__ expert_base,
    const uint32_t* __restrict__ before_me, ByteTable recv_packed, ByteTable recv_scales, WordTable recv_origin, uint32_t routes,
    uint32_t routes_per_row, uint32_t k, uint32_t tile_bytes, uint32_t experts, uint32_t world, uint32_t rank) {
    const uint32_t sorted = blockIdx.x * kDispatchWarps + (threadIdx.x >> 5);
    const uint32_t lane = threadIdx.x & 31;
    if (sorted >= routes) return;
    const uint32_t route = sorted_routes[sorted];
    const uint32_t expert = sorted_experts[sorted];
    if (expert >= experts) return;
    const uint32_t per = experts / world;
    const uint32_t owner = expert / per, local_expert = expert - owner * per;
    const uint32_t col = before_me[expert] + (sorted - local_offsets[expert]);  // row inside the expert at the owner
    const uint32_t base = expert_base[expert];
    const uint32_t dst_row = base + col;
    const uint32_t src_row = route / routes_per_row;
    const uint32_t row_bytes = k / 2;  // a multiple of 16 (k % 32 == 0 is checked on the host)
    const uint4* s4 = reinterpret_cast<const uint4*>(src_packed + static_cast<size_t>(src_row) * row_bytes);
    uint4* d4 = reinterpret_cast<uint4*>(recv_packed.p[owner] + static_cast<size_t>(dst_row) * row_bytes);
    for (uint32_t i = lane; i < row_bytes / 16; i += 32) d4[i] = __ldg(s4 + i);
    // scale bytes: four consecutive blocks of a row are one aligned 4-byte word in both tile layouts
    uint8_t* scales = recv_scales.p[owner] + ((static_cast<size_t>(base) + 127) / 128 + local_expert) * tile_bytes;
    const uint32_t blocks = k / 16;
    for (uint32_t w = lane; w < blocks / 4; w += 32)
        *reinterpret_cast<uint32_t*>(scales + tiled_scale_offset(col, w * 4, k)) =
            __ldg(reinterpret_cast<const uint32_t*>(src_scales + tiled_scale_offset(src_row, w * 4, k)));
    for (uint32_t b = (blocks / 4) * 4 + lane; b < blocks; b += 32)
        scales[tiled_scale_offset(col, b, k)] = __ldg(src_scales + tiled_scale_offset(src_row, b, k));
    if (lane == 0) recv_origin.p[owner][dst_row] = (rank << 24) | route;
}

// sorted_experts[row] for the rows a rank received: the expert whose offset range holds the row; rows past the total get
// `per` (no expert) so that later kernels skip them.
__global__ void __launch_bounds__(256) ep_expand_experts_kernel(const uint32_t* __restrict__ recv_offsets, uint32_t per,
                                                                uint32_t* __restrict__ sorted_experts, uint32_t capacity) {
    const uint32_t row = blockIdx.x * blockDim.x + threadIdx.x;
    if (row >= capacity) return;
    uint32_t lo = 0, hi = per;  // first e with offsets[e + 1] > row
    while (lo < hi) {
        const uint32_t mid = (lo + hi) / 2;
        if (recv_offsets[mid + 1] > row) hi = mid;
        else lo = mid + 1;
    }
    sorted_experts[row] = lo;
}

// The bf16 result rows go back to the source rank of their route, at the route's own index.  Each row is one contiguous
// run of 2 * n bytes on both sides, so it travels as two bulk copies of the copy engine: global -> shared memory (completes
// on an mbarrier), shared memory -> the peer's return buffer.  NVLink then carries whole rows in full-size packets, which
// plain 16-byte stores per lane did not (about 390 GB/s).  One row per warp at a time, persistent warps; every wait is
// bounded and a warp that gives up simply stops copying (the layer's status shows up as wrong rows in no case: the host
// checks the barrier status, and the bound is a second).
constexpr uint32_t kReturnWarps = 4;

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__global__ void __launch_bounds__(kReturnWarps * 32) ep_return_rows_kernel(const uint16_t* __restrict__ rows,
                                                                           const uint32_t* __restrict__ origin,
                                                                           const uint32_t* __restrict__ recv_total, ByteTable ret,
                                                                           uint32_t capacity, uint32_t n) {
    extern __shared__ __align__(128) uint8_t stage[];  // [kReturnWarps][2 * n]
    __shared__ __align__(8) uint64_t bars[kReturnWarps];
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t row_bytes = n * 2;
    if (lane != 0) return;  // one thread per warp drives the copy engine
    const uint32_t bar = smem_addr(&bars[warp]);
    const uint32_t buf = smem_addr(stage + static_cast<size_t>(warp) * row_bytes);
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    const uint32_t total = min(capacity, recv_total[0]);
    uint32_t phase = 0;
    for (uint32_t row = blockIdx.x * kReturnWarps + warp; row < total; row += gridDim.x * kReturnWarps) {
        // the store that last read this buffer has finished reading it
        asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(row_bytes) : "memory");
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(buf),
                     "l"(rows + static_cast<size_t>(row) * n), "r"(row_bytes), "r"(bar)
                     : "memory");
        const long long start = clock64();
        uint32_t done = 0;
        while (!done) {
            asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
                         : "=r"(done) : "r"(bar), "r"(phase) : "memory");
            if (!done && clock64() - start > 2000000000ll) return;
        }
        phase ^= 1;
        const uint32_t o = origin[row];
        uint8_t* dst = ret.p[o >> 24] + static_cast<size_t>(o & 0xffffffu) * row_bytes;
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(buf), "r"(row_bytes) : "memory");
        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
    }
    asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");  // the rows have left before the kernel (and the barrier behind it) ends
}

}  // namespace
}  // namespace eider

using namespace eider;

extern "C" {

size_t eider_b200_peer_barrier_pad_bytes(void) { return kChannels * kMaxRanks * sizeof(uint32_t); }
size_t eider_b200_peer_barrier_state_bytes(void) { return (kChannels + 1) * sizeof(uint32_t); }

cudaError_t eider_b200_peer_barrier_on_stream(void* const* signal_pads, uint32_t world, uint32_t rank, uint32_t channel,
                                              uint32_t* state, uint64_t timeout_cycles, cudaStream_t stream) {
    if (!signal_pads || !state || world == 0 || world > kMaxRanks || rank >= world || channel >= kChannels)
        return cudaErrorInvalidValue;
    PadTable pads{};
    for (uint32_t q = 0; q < world; ++q) {
        if (!signal_pads[q] || (reinterpret_cast<uintptr_t>(signal_pads[q]) & 3) != 0) return cudaErrorInvalidValue;
        pads.pad[q] = static_cast<uint32_t*>(signal_pads[q]);
    }
    if (timeout_cycles == 0) timeout_cycles = 2000000000ull;  // about a second of SM clock
    peer_barrier_kernel<<<1, 32, 0, stream>>>(pads, world, rank, channel, state, static_cast<long long>(timeout_cycles));
    return cudaGetLastError();
}

static bool fill_bytes(ByteTable& t, void* const* ptrs, uint32_t world, uintptr_t align_mask) {
    if (!ptrs) return false;
    for (uint32_t q = 0; q < world; ++q) {
        if (!ptrs[q] || (reinterpret_cast<uintptr_t>(ptrs[q]) & align_mask) != 0) return false;
        t.p[q] = static_cast<uint8_t*>(ptrs[q]);
    }
    return true;
}
static bool fill_words(WordTable& t, void* const* ptrs, uint32_t world) {
    if (!ptrs) return false;
    for (uint32_t q = 0; q < world; ++q) {
        if (!ptrs[q] || (reinterpret_cast<uintptr_t>(ptrs[q]) & 3) != 0) return false;
        t.p[q] = static_cast<uint32_t*>(ptrs[q]);
    }
    return true;
}

cudaError_t eider_b200_ep_publish_counts_on_stream(const uint32_t* expert_counts, void* const* counts_all, uint32_t world,
                                                   uint32_t rank, uint32_t experts, cudaStream_t stream) {
    WordTable t{};
    if (!expert_counts || world == 0 || world > kMaxRanks || rank >= world || experts == 0 || !fill_words(t, counts_all, world))
        return cudaErrorInvalidValue;
    ep_publish_counts_kernel<<<(experts + 127) / 128, 128, 0, stream>>>(expert_counts, t, world, rank, experts);
    return cudaGetLastError();
}

cudaError_t eider_b200_ep_offsets_on_stream(const uint32_t* counts_all, uint32_t world, uint32_t rank, uint32_t experts,
                                            uint32_t* expert_base, uint32_t* before_me, uint32_t* recv_offsets,
                                            uint32_t* recv_total, cudaStream_t stream) {
    if (!counts_all || !expert_base || !before_me || !recv_offsets || !recv_total || world == 0 || world > kMaxRanks ||
        rank >= world || experts == 0 || experts > 1024 || experts % world != 0)
        return cudaErrorInvalidValue;
    ep_offsets_kernel<<<1, 1024, 0, stream>>>(counts_all, world, rank, experts, expert_base, before_me, recv_offsets, recv_total);
    return cudaGetLastError();
}

cudaError_t eider_b200_ep_dispatch_rows_on_stream(const uint8_t* source_packed, const uint8_t* source_scales,
                                                  const uint32_t* sorted_routes, const uint32_t* sorted_experts,
                                                  const uint32_t* local_offsets, const uint32_t* expert_base,
                                                  const uint32_t* before_me, void* const* recv_packed, void* const* recv_scales,
                                                  void* const* recv_origin, uint32_t routes, uint32_t routes_per_row,
                                                  uint32_t in_features, uint32_t scale_tile_bytes, uint32_t experts, uint32_t world,
                                                  uint32_t rank, cudaStream_t stream) {
    ByteTable packed{}, scales{};
    WordTable origin{};
    if (!source_packed || !source_scales || !sorted_routes || !sorted_experts || !local_offsets || !expert_base || !before_me ||
        routes == 0 || routes >= (1u << 24) || routes_per_row == 0 || in_features == 0 || in_features % 32 != 0 ||
        scale_tile_bytes == 0 || world == 0 || world > kMaxRanks || rank >= world || experts % world != 0 ||
        (reinterpret_cast<uintptr_t>(source_packed) & 15) != 0 || (reinterpret_cast<uintptr_t>(source_scales) & 3) != 0 ||
        !fill_bytes(packed, recv_packed, world, 15) || !fill_bytes(scales, recv_scales, world, 3) || !fill_words(origin, recv_origin, world))
        return cudaErrorInvalidValue;
    ep_dispatch_rows_kernel<<<(routes + kDispatchWarps - 1) / kDispatchWarps, kDispatchWarps * 32, 0, stream>>>(
        source_packed, source_scales, sorted_routes, sorted_experts, local_offsets, expert_base, before_me, packed, scales, origin,
        routes, routes_per_row, in_features, scale_tile_bytes, experts, world, rank);
    return cudaGetLastError();
}

cudaError_t eider_b200_ep_expand_experts_on_stream(const uint32_t* recv_offsets, uint32_t local_experts, uint32_t* sorted_experts,
                                                   uint32_t capacity, cudaStream_t stream) {
    if (!recv_offsets || !sorted_experts || local_experts == 0 || capacity == 0) return cudaErrorInvalidValue;
    ep_expand_experts_kernel<<<(capacity + 255) / 256, 256, 0, stream>>>(recv_offsets, local_experts, sorted_experts, capacity);
    return cudaGetLastError();
}

cudaError_t eider_b200_ep_return_rows_on_stream(const uint16_t* rows, const uint32_t* recv_origin, const uint32_t* recv_total,
                                                void* const* return_rows, uint32_t capacity, uint32_t out_features, uint32_t world,
                                                cudaStream_t stream) {
    ByteTable ret{};
    if (!rows || !recv_origin || !recv_total || capacity == 0 || out_features == 0 || out_features % 8 != 0 || world == 0 ||
        world > kMaxRanks || (reinterpret_cast<uintptr_t>(rows) & 15) != 0 || !fill_bytes(ret, return_rows, world, 15))
        return cudaErrorInvalidValue;
    const size_t smem = static_cast<size_t>(kReturnWarps) * out_features * 2;
    if (smem > 160 * 1024) return cudaErrorNotSupported;
    if (smem > 48 * 1024) {
        cudaError_t st = cudaFuncSetAttribute(ep_return_rows_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        if (st != cudaSuccess) return st;
    }
    // persistent warps: enough CTAs to fill the machine, never more than there are rows
    uint32_t grid = (capacity + kReturnWarps - 1) / kReturnWarps;
    if (grid > 148 * 8) grid = 148 * 8;
    ep_return_rows_kernel<<<grid, kReturnWarps * 32, smem, stream>>>(rows, recv_origin, recv_total, ret, capacity, out_features);
    return cudaGetLastError();
}

}  // extern "C"
