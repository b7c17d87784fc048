// Routed-MoE data movement around the grouped GEMM: router top-k, route permutation (expert-major order),
// gather + NVFP4 quantize into per-expert scale tiles, SiLU(gate) * up + quantize, pointer tables, and the
// weighted un-permute.  HBM-bound integer / byte work; every kernel is sized so consecutive lanes touch
// consecutive bytes and each token is quantized once.
//
// Semantics follow crates/eider-cuda/native/non_gemm.cu (lines cited per kernel).
#include "common.cuh"
#include "rowops.cuh"
#include "eider_b200.h"

namespace eider {
namespace {

constexpr uint32_t kFull = 0xffffffffu;

__device__ __forceinline__ float sanitize_logit(float v) {
    // non_gemm.cu:1876-1881: NaN -> -inf, +inf -> FLT_MAX
    if (v != v) return -INFINITY;
    if (v == INFINITY) return 3.402823466e+38f;
    return v;
}

// Router top-k, one warp per token (non_gemm.cu:1854-2020).  Selection = k rounds of "largest value, lowest
// expert index on ties", which is the order the reference's strict-'>' insertion produces.
template <int PER_LANE>
__global__ void __launch_bounds__(128) moe_topk_kernel(const float* __restrict__ logits, uint32_t* __restrict__ out_idx,
                                                       float* __restrict__ out_w, uint32_t tokens, uint32_t experts,
                                                       uint32_t k, int norm_topk_prob) {
    const uint32_t token = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (token >= tokens) return;
    const uint32_t lane = threadIdx.x & 31;
    const float* lg = logits + static_cast<size_t>(token) * experts;
    uint32_t* idx = out_idx + static_cast<size_t>(token) * k;
    float* w = out_w + static_cast<size_t>(token) * k;
    float v[PER_LANE];
    float mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < PER_LANE; ++i) {
        const uint32_t e = lane + i * 32;
        v[i] = e < experts ? sanitize_logit(__ldg(lg + e)) : -INFINITY;
        mx = fmaxf(mx, v[i]);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(kFull, mx, o));
    if (!(fabsf(mx) < INFINITY)) {  // every logit non-finite: expert 0 with weight 1 (non_gemm.cu:1889-1895, 1945-1953)
        for (uint32_t s = lane; s < k; s += 32) {
            idx[s] = s;
            w[s] = s == 0 ? 1.0f : 0.0f;
        }
        return;
    }
    if (!norm_topk_prob) {
        // full softmax first, then top-k of the probabilities (non_gemm.cu:1913-2005)
        float sum = 0.0f;
#pragma unroll
        for (int i = 0; i < PER_LANE; ++i) {
            const uint32_t e = lane + i * 32;
            v[i] = e < experts ? expf(v[i] - mx) : -INFINITY;
            if (e < experts) sum += v[i];
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(kFull, sum, o);
#pragma unroll
        for (int i = 0; i < PER_LANE; ++i)
            if (lane + i * 32 < experts) v[i] = __fdiv_rn(v[i], sum);
    }
    float sel_first = 0.0f, sel_sum = 0.0f, my_w = 0.0f;
    for (uint32_t s = 0; s < k; ++s) {
        float best = -INFINITY;
        uint32_t best_e = 0xffffffffu;
#pragma unroll
        for (int i = 0; i < PER_LANE; ++i) {
            const uint32_t e = lane + i * 32;
            if (e < experts && (v[i] > best || (v[i] == best && e < best_e))) {
                best = v[i];
                best_e = e;
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(kFull, best, o);
            const uint32_t oe = __shfl_xor_sync(kFull, best_e, o);
            if (ob > best || (ob == best && oe < best_e)) {
                best = ob;
                best_e = oe;
            }
        }
        // remove the winner from its owner's candidates
#pragma unroll
        for (int i = 0; i < PER_LANE; ++i)
            if (lane + i * 32 == best_e) v[i] = -INFINITY;
        float weight = best;
        if (norm_topk_prob) {
            if (s == 0) sel_first = best;
            weight = expf(best - sel_first);  // softmax over the selected logits (non_gemm.cu:1897-1909)
            sel_sum += weight;
        }
        if (lane == (s & 31)) my_w = weight;  // slot s is kept by lane s % 32 (k <= 32)
        if (lane == 0) idx[s] = best_e;
    }
    if (norm_topk_prob && sel_sum > 0.0f && fabsf(sel_sum) < INFINITY) my_w = __fdiv_rn(my_w, sel_sum);
    if (lane < k) w[lane] = my_w;
}

// ---- route permutation ------------------------------------------------------------------------------
constexpr uint32_t kSortChunk = 256;

// per-chunk histogram of expert ids
__global__ void __launch_bounds__(kSortChunk) moe_chunk_hist_kernel(const uint32_t* __restrict__ indices,
                                                                   uint32_t* __restrict__ chunk_hist, uint32_t routes,
                                                                   uint32_t experts) {
    extern __shared__ uint32_t hist[];
    for (uint32_t e = threadIdx.x; e < experts; e += blockDim.x) hist[e] = 0;
    __syncthreads();
    const uint32_t r = blockIdx.x * kSortChunk + threadIdx.x;
    if (r < routes) {
        const uint32_t e = __ldg(indices + r);
        if (e < experts) atomicAdd(&hist[e], 1u);
    }
    __syncthreads();
    for (uint32_t e = threadIdx.x; e < experts; e += blockDim.x) chunk_hist[static_cast<size_t>(blockIdx.x) * experts + e] = hist[e];
}

// Exclusive prefix over chunks per expert (in place), totals, then a block scan over experts.  The chunk range of an
// expert is split over 1024 / experts threads: each sums its segment with independent loads, the segment bases come from
// shared memory, and a second pass over the (cache-resident) segment writes the prefixes; the dependent chain is a few
// loads long instead of one load per chunk.
__global__ void __launch_bounds__(1024) moe_prefix_kernel(uint32_t* __restrict__ chunk_hist, uint32_t* __restrict__ counts,
                                                          uint32_t* __restrict__ offsets, uint32_t* __restrict__ cursors,
                                                          uint32_t chunks, uint32_t experts) {
    __shared__ uint32_t scan[1024];
    __shared__ uint32_t partial[1024];
    const uint32_t parts = 1024 / experts;  // experts <= 1024 is checked on the host
    const uint32_t e = threadIdx.x % experts;
    const uint32_t part = threadIdx.x / experts;
    const bool active = part < parts;
    const uint32_t seg = (chunks + parts - 1) / parts;
    const uint32_t c0 = min(chunks, part * seg), c1 = min(chunks, c0 + seg);
    uint32_t sum = 0;
    if (active) {
        uint32_t c = c0;
        for (; c + 8 <= c1; c += 8) {
            uint32_t h[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) h[i] = chunk_hist[static_cast<size_t>(c + i) * experts + e];
#pragma unroll
            for (int i = 0; i < 8; ++i) sum += h[i];
        }
        for (; c < c1; ++c) sum += chunk_hist[static_cast<size_t>(c) * experts + e];
        partial[part * experts + e] = sum;
    }
    __syncthreads();
    uint32_t running = 0, total = 0;
    if (active) {
        for (uint32_t q = 0; q < parts; ++q) {
            const uint32_t v = partial[q * experts + e];
            if (q < part) running += v;
            total += v;
        }
        uint32_t c = c0;
        for (; c + 8 <= c1; c += 8) {
            uint32_t h[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) h[i] = chunk_hist[static_cast<size_t>(c + i) * experts + e];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                chunk_hist[static_cast<size_t>(c + i) * experts + e] = running;
                running += h[i];
            }
        }
        for (; c < c1; ++c) {
            const uint32_t h = chunk_hist[static_cast<size_t>(c) * experts + e];
            chunk_hist[static_cast<size_t>(c) * experts + e] = running;
            running += h;
        }
    }
    // scan over experts (threads 0 .. experts-1 hold the totals)
    const uint32_t t = threadIdx.x;
    const bool owner = t < experts;  // part == 0, e == t
    if (owner) counts[t] = total;
    scan[t] = owner ? total : 0;
    __syncthreads();
    for (uint32_t o = 1; o < 1024; o <<= 1) {  // Hillis-Steele inclusive scan
        const uint32_t add = t >= o ? scan[t - o] : 0;
        __syncthreads();
        scan[t] += add;
        __syncthreads();
    }
    if (owner) {
        const uint32_t excl = scan[t] - total;
        offsets[t] = excl;
        cursors[t] = excl + total;  // where the reference's atomic cursor ends up (non_gemm.cu:2511)
    }
    if (t == experts - 1) offsets[experts] = scan[t];
}

// stable scatter: routes of one expert keep ascending route order
__global__ void __launch_bounds__(kSortChunk) moe_scatter_kernel(const uint32_t* __restrict__ indices,
                                                                const uint32_t* __restrict__ chunk_base,
                                                                const uint32_t* __restrict__ offsets,
                                                                uint32_t* __restrict__ sorted_routes,
                                                                uint32_t* __restrict__ sorted_experts,
                                                                uint32_t* __restrict__ route_to_sorted, uint32_t routes,
                                                                uint32_t experts) {
    extern __shared__ uint32_t wcount[];  // [warps][experts]
    constexpr uint32_t kWarps = kSortChunk / 32;
    for (uint32_t i = threadIdx.x; i < kWarps * experts; i += blockDim.x) wcount[i] = 0;
    __syncthreads();
    const uint32_t r = blockIdx.x * kSortChunk + threadIdx.x;
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t e = r < routes ? __ldg(indices + r) : 0xffffffffu;
    const bool valid = e < experts;
    const uint32_t peers = __match_any_sync(kFull, valid ? e : 0xffffffffu);
    const uint32_t rank = __popc(peers & ((1u << lane) - 1));
    if (valid && rank == 0) wcount[warp * experts + e] = __popc(peers);
    __syncthreads();
    if (!valid) return;
    uint32_t before = 0;
    for (uint32_t w = 0; w < warp; ++w) before += wcount[w * experts + e];
    const uint32_t sorted = offsets[e] + chunk_base[static_cast<size_t>(blockIdx.x) * experts + e] + before + rank;
    sorted_routes[sorted] = r;
    sorted_experts[sorted] = e;
    route_to_sorted[r] = sorted;
}

// non_gemm.cu:2554-2557: one spare 128-row scale tile per expert around the sorted prefix
__device__ __forceinline__ size_t moe_scale_base(uint32_t expert, const uint32_t* offsets, uint32_t tile_bytes) {
    return ((static_cast<size_t>(offsets[expert]) + 127) / 128 + expert) * tile_bytes;
}

// Scatter already quantized token rows into expert-major order (second half of non_gemm.cu:2899-2998).  One warp per
// sorted route: packed bytes move 16 at a time, the row's scale bytes move as the 4-byte words they form in the 128 x 4
// tile layout (four consecutive blocks of a row are adjacent in both the token-tiled source and the expert's tiles).
constexpr uint32_t kScatterWarps = 8;
__global__ void __launch_bounds__(kScatterWarps * 32) moe_scatter_rows_kernel(const uint8_t* __restrict__ src_packed,
                                                                              const uint8_t* __restrict__ src_scales,
                                                                              const uint32_t* __restrict__ sorted_routes,
                                                                              const uint32_t* __restrict__ sorted_experts,
                                                                              const uint32_t* __restrict__ offsets,
                                                                              uint8_t* __restrict__ packed,
                                                                              uint8_t* __restrict__ scales, uint32_t routes,
                                                                              uint32_t routes_per_row, uint32_t k,
                                                                              uint32_t tile_bytes, int gather_rows) {
    const uint32_t sorted = blockIdx.x * kScatterWarps + (threadIdx.x >> 5);
    const uint32_t lane = threadIdx.x & 31;
    if (sorted >= routes) return;
    const uint32_t src_row = gather_rows ? sorted_routes[sorted] / routes_per_row : sorted;
    const uint32_t expert = sorted_experts[sorted];
    const uint32_t col = sorted - offsets[expert];
    const uint32_t row_bytes = k / 2;
    const uint8_t* s1 = src_packed + static_cast<size_t>(src_row) * row_bytes;
    uint8_t* d1 = packed + static_cast<size_t>(sorted) * row_bytes;
    if (row_bytes % 16 == 0 && ((reinterpret_cast<uintptr_t>(src_packed) | reinterpret_cast<uintptr_t>(packed)) & 15) == 0) {
        const uint4* s4 = reinterpret_cast<const uint4*>(s1);
        uint4* d4 = reinterpret_cast<uint4*>(d1);
        for (uint32_t i = lane; i < row_bytes / 16; i += 32) d4[i] = __ldg(s4 + i);
    } else {  // rows that do not start on 16-byte boundaries (K % 32 != 0): 8-byte words, K % 16 == 0 guarantees those
        const uint2* s2 = reinterpret_cast<const uint2*>(s1);
        uint2* d2 = reinterpret_cast<uint2*>(d1);
        for (uint32_t i = lane; i < row_bytes / 8; i += 32) d2[i] = __ldg(s2 + i);
    }
    const size_t base = moe_scale_base(expert, offsets, tile_bytes);
    const uint32_t blocks = k / 16;
    const bool aligned4 = ((reinterpret_cast<uintptr_t>(scales) | reinterpret_cast<uintptr_t>(src_scales)) & 3) == 0;
    const uint32_t words = aligned4 ? blocks / 4 : 0;  // whole groups of four blocks
    for (uint32_t w = lane; w < words; w += 32)
        *reinterpret_cast<uint32_t*>(scales + base + tiled_scale_offset(col, w * 4, k)) =
            __ldg(reinterpret_cast<const uint32_t*>(src_scales + tiled_scale_offset(src_row, w * 4, k)));
    for (uint32_t b = words * 4 + lane; b < blocks; b += 32)
        scales[base + tiled_scale_offset(col, b, k)] = __ldg(src_scales + tiled_scale_offset(src_row, b, k));
}

// silu(gate) * up on bf16 halves, then NVFP4 with unit global scale into the expert's scale tiles
// (non_gemm.cu:2805-2875).  One thread per 8 products, two neighbouring threads share a 16-element block; the grid is
// flat over all routes so that a CTA is full whatever the row length.
__global__ void __launch_bounds__(256) moe_silu_mul_quantize_kernel(const uint16_t* __restrict__ gate_up,
                                                                    const uint32_t* __restrict__ sorted_experts,
                                                                    const uint32_t* __restrict__ offsets,
                                                                    uint8_t* __restrict__ packed, uint8_t* __restrict__ scales,
                                                                    uint32_t routes, uint32_t k, uint32_t tile_bytes,
                                                                    const uint32_t* __restrict__ routes_limit) {
    const uint32_t halves = k / 8;
    const uint64_t unit = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    // (routes_limit: optional device-resident row count below the launch's capacity, for buffers filled by other ranks)
    const bool live = unit < static_cast<uint64_t>(routes) * halves && (!routes_limit || unit / halves < __ldg(routes_limit));
    const uint32_t sorted = live ? static_cast<uint32_t>(unit / halves) : 0;
    const uint32_t h = live ? static_cast<uint32_t>(unit % halves) : 0;
    float v[8];
    float amax = 0.0f;
    if (live) {
        const uint16_t* gate = gate_up + static_cast<size_t>(sorted) * k * 2;
        const uint16_t* up = gate + k;
        const uint4 g4 = __ldg(reinterpret_cast<const uint4*>(gate + h * 8));
        const uint4 u4 = __ldg(reinterpret_cast<const uint4*>(up + h * 8));
        const uint32_t gw[4] = {g4.x, g4.y, g4.z, g4.w}, uw[4] = {u4.x, u4.y, u4.z, u4.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float g0 = __uint_as_float(gw[j] << 16), g1 = __uint_as_float(gw[j] & 0xffff0000u);
            const float u0 = __uint_as_float(uw[j] << 16), u1 = __uint_as_float(uw[j] & 0xffff0000u);
            v[2 * j] = moe_silu_mul(g0, u0);
            v[2 * j + 1] = moe_silu_mul(g1, u1);
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) amax = fmaxf(amax, finite_abs(v[i]));
    }
    // k / 8 is even, so the two halves of a block are lanes 2i and 2i + 1 of one warp and belong to one route
    amax = fmaxf(amax, __shfl_xor_sync(kFull, amax, 1));
    if (!live) return;
    const uint8_t sc = amax == 0.0f ? 0 : ue4m3_code(div6_rn(amax));
    const float sv = e4m3_value(sc);
    const Divisor ds = make_divisor(sv == 0.0f ? 1.0f : sv);
    uint32_t w = 0;
#pragma unroll
    for (int i = 0; i < 8; i += 2) {
        const float lo = sv == 0.0f ? 0.0f : div_rn(v[i], ds);
        const float hi = sv == 0.0f ? 0.0f : div_rn(v[i + 1], ds);
        w |= static_cast<uint32_t>(e2m1x2_code(lo, hi)) << (i * 4);
    }
    *reinterpret_cast<uint32_t*>(packed + static_cast<size_t>(sorted) * (k / 2) + h * 4) = w;
    if ((h & 1) == 0) {
        const uint32_t expert = sorted_experts[sorted];
        scales[moe_scale_base(expert, offsets, tile_bytes) + tiled_scale_offset(sorted - offsets[expert], h >> 1, k)] = sc;
    }
}

// Quantize sorted rows straight from their source, one thread per 16-element block, grid flat over routes x blocks.
// The source row and the value formula depend on MODE:
//   kPlain       f32 rows, row = gather ? sorted_routes[sorted] / routes_per_row : sorted          (non_gemm.cu:2621-2676)
//   kCalibrated  the same rows times 1 / input_scales[expert]                                      (non_gemm.cu:2562-2600)
//   kReluSquared sorted bf16 rows: max(x, 0)^2 times 1 / input_scales[expert]                      (same kernel)
//   kGeluPair    sorted bf16 gate and up rows: GELU-tanh(gate) * up                                (non_gemm.cu:2705-2780)
enum SortedQuantMode { kPlain = 0, kCalibrated = 1, kReluSquared = 2, kGeluPair = 3 };

template <int MODE>
__global__ void __launch_bounds__(256) moe_quantize_sorted_kernel(const void* __restrict__ input, const void* __restrict__ input2,
                                                                  const float* __restrict__ input_scales,
                                                                  const uint32_t* __restrict__ sorted_routes,
                                                                  const uint32_t* __restrict__ sorted_experts,
                                                                  const uint32_t* __restrict__ offsets, uint8_t* __restrict__ packed,
                                                                  uint8_t* __restrict__ scales, uint32_t routes,
                                                                  uint32_t routes_per_row, uint32_t k, uint32_t tile_bytes,
                                                                  int gather_rows) {
    const uint32_t blocks = k / 16;
    const uint64_t unit = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (unit >= static_cast<uint64_t>(routes) * blocks) return;
    const uint32_t sorted = static_cast<uint32_t>(unit / blocks), b = static_cast<uint32_t>(unit % blocks);
    const uint32_t expert = __ldg(sorted_experts + sorted);
    float v[16];
    if (MODE == kPlain || MODE == kCalibrated) {
        const uint32_t src_row = gather_rows ? __ldg(sorted_routes + sorted) / routes_per_row : sorted;
        const float* src = static_cast<const float*>(input) + static_cast<size_t>(src_row) * k + b * 16;
        const float inverse = MODE == kCalibrated ? __frcp_rn(__ldg(input_scales + expert)) : 1.0f;
#pragma unroll
        for (int i = 0; i < 16; ++i) v[i] = MODE == kCalibrated ? __fmul_rn(__ldg(src + i), inverse) : __ldg(src + i);
    } else {
        const uint16_t* src = static_cast<const uint16_t*>(input) + static_cast<size_t>(sorted) * k + b * 16;
        if (MODE == kReluSquared) {
            const float inverse = __frcp_rn(__ldg(input_scales + expert));
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const float x = fmaxf(bf16_bits_to_float(__ldg(src + i)), 0.0f);
                v[i] = __fmul_rn(__fmul_rn(x, x), inverse);
            }
        } else {
            const uint16_t* up = static_cast<const uint16_t*>(input2) + static_cast<size_t>(sorted) * k + b * 16;
#pragma unroll
            for (int i = 0; i < 16; ++i) v[i] = rowops::gelu_tanh_mul(bf16_bits_to_float(__ldg(src + i)), bf16_bits_to_float(__ldg(up + i)));
        }
    }
    uint2 bytes;
    const uint8_t sc = quantize_block16(v, 16, &bytes);
    uint8_t* dst = packed + static_cast<size_t>(sorted) * (k / 2) + b * 8;  // 8-byte aligned when `packed` is (k % 16 == 0)
    *reinterpret_cast<uint2*>(dst) = bytes;
    scales[moe_scale_base(expert, offsets, tile_bytes) + tiled_scale_offset(sorted - __ldg(offsets + expert), b, k)] = sc;
}

// non_gemm.cu:3066-3083
__global__ void moe_pointer_tables_kernel(const uint32_t* __restrict__ offsets, const uint8_t* packed, const uint8_t* scales,
                                          uint16_t* output, const uint8_t** packed_table, const uint8_t** scale_table,
                                          uint16_t** output_table, uint32_t experts, uint32_t in_features,
                                          uint32_t out_features, uint32_t tile_bytes) {
    const uint32_t e = blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= experts) return;
    const size_t off = offsets[e];
    packed_table[e] = packed + off * (in_features / 2);
    scale_table[e] = scales + moe_scale_base(e, offsets, tile_bytes);
    output_table[e] = output + off * out_features;
}

// Un-permute + weighted sum in slot order (non_gemm.cu:3735-3758): out[t][c] = sum_slot bf16(y[inv[t*k+slot]][c]) * w.
// One thread per 8 output columns: 128-bit loads of the sorted rows, two 128-bit stores.
__global__ void __launch_bounds__(256) moe_combine_kernel(const uint32_t* __restrict__ route_to_sorted,
                                                          const float* __restrict__ route_weights,
                                                          const uint16_t* __restrict__ sorted_inputs, float* __restrict__ output,
                                                          uint32_t rows, uint32_t len, uint32_t routes_per_row) {
    const uint32_t vec_per_row = len / 8;
    const size_t idx = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= static_cast<size_t>(rows) * vec_per_row) return;
    const uint32_t row = static_cast<uint32_t>(idx / vec_per_row), v = static_cast<uint32_t>(idx % vec_per_row);
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (uint32_t slot = 0; slot < routes_per_row; ++slot) {
        const uint32_t route = row * routes_per_row + slot;
        const uint32_t sorted = __ldg(route_to_sorted + route);
        const float w = __ldg(route_weights + route);
        const uint4 q = __ldg(reinterpret_cast<const uint4*>(sorted_inputs + static_cast<size_t>(sorted) * len) + v);
        const uint32_t ww[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            acc[2 * j] = fmaf(__uint_as_float(ww[j] << 16), w, acc[2 * j]);
            acc[2 * j + 1] = fmaf(__uint_as_float(ww[j] & 0xffff0000u), w, acc[2 * j + 1]);
        }
    }
    float4* dst = reinterpret_cast<float4*>(output + static_cast<size_t>(row) * len + v * 8);
    dst[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
    dst[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
}

__global__ void __launch_bounds__(256) moe_combine_scalar_kernel(const uint32_t* __restrict__ route_to_sorted,
                                                                 const float* __restrict__ route_weights,
                                                                 const uint16_t* __restrict__ sorted_inputs,
                                                                 float* __restrict__ output, uint32_t rows, uint32_t len,
                                                                 uint32_t routes_per_row) {
    const size_t idx = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= static_cast<size_t>(rows) * len) return;
    const uint32_t row = static_cast<uint32_t>(idx / len), col = static_cast<uint32_t>(idx % len);
    float sum = 0.0f;
    for (uint32_t slot = 0; slot < routes_per_row; ++slot) {
        const uint32_t route = row * routes_per_row + slot;
        sum = fmaf(bf16_bits_to_float(sorted_inputs[static_cast<size_t>(route_to_sorted[route]) * len + col]),
                   route_weights[route], sum);
    }
    output[idx] = sum;
}

}  // namespace
}  // namespace eider

// ---- scratch for the entry point that must not allocate ------------------------------------------------
// Fixed-size chunk-histogram table for eider_b200_moe_sort_routes_noalloc_on_stream.  It lives in every GPU context
// that loads the library (1 MiB) until the process exits.  In host code the name below is only a handle: kernels must
// be given the device address that cudaGetSymbolAddress returns for the current device.
namespace eider {
namespace {
constexpr uint32_t kNoAllocSortEntries = 262144;  // chunks * experts, 4 bytes each
static __device__ __align__(256) uint32_t g_noalloc_sort_scratch[kNoAllocSortEntries];

constexpr int kMaxDevices = 64;
uint32_t* g_noalloc_sort_ptr[kMaxDevices] = {nullptr};

// Device address of the scratch table on the current device, looked up once per device.
cudaError_t noalloc_sort_scratch(uint32_t** out) {
    int dev = -1;
    cudaError_t st = cudaGetDevice(&dev);
    if (st != cudaSuccess) return st;
    if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
    if (g_noalloc_sort_ptr[dev] == nullptr) {
        uint32_t* ptr = nullptr;
        st = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_noalloc_sort_scratch);
        if (st != cudaSuccess) return st;
        g_noalloc_sort_ptr[dev] = ptr;
    }
    *out = g_noalloc_sort_ptr[dev];
    return cudaSuccess;
}
}  // namespace
}  // namespace eider

using namespace eider;

extern "C" {

cudaError_t infer_moe_topk_f32_batch_on_stream(const float* logits, uint32_t* out_indices, float* out_weights,
                                               uint32_t batch_size, uint32_t experts, uint32_t k, int norm_topk_prob,
                                               cudaStream_t stream) {
    if (!logits || !out_indices || !out_weights || batch_size == 0 || experts == 0 || k == 0 || k > experts || k > 32 ||
        experts > 1024)
        return cudaErrorInvalidValue;
    const uint32_t grid = (batch_size + 3) / 4;
    const uint32_t per_lane = (experts + 31) / 32;
#define EIDER_TOPK(P) moe_topk_kernel<P><<<grid, 128, 0, stream>>>(logits, out_indices, out_weights, batch_size, experts, k, norm_topk_prob)
    if (per_lane <= 1) EIDER_TOPK(1);
    else if (per_lane <= 2) EIDER_TOPK(2);
    else if (per_lane <= 4) EIDER_TOPK(4);
    else if (per_lane <= 8) EIDER_TOPK(8);
    else if (per_lane <= 16) EIDER_TOPK(16);
    else EIDER_TOPK(32);
#undef EIDER_TOPK
    return cudaGetLastError();
}

cudaError_t infer_moe_topk_f32_on_stream(const float* logits, uint32_t* out_indices, float* out_weights, uint32_t experts,
                                         uint32_t k, int norm_topk_prob, cudaStream_t stream) {
    return infer_moe_topk_f32_batch_on_stream(logits, out_indices, out_weights, 1, experts, k, norm_topk_prob, stream);
}

size_t eider_b200_moe_sort_scratch_bytes(uint32_t routes, uint32_t experts) {
    return static_cast<size_t>((routes + kSortChunk - 1) / kSortChunk) * experts * sizeof(uint32_t);
}

// The three launches of the stable route sort over a chunk-histogram table of ceil(routes / 256) * experts words.
static cudaError_t sort_routes_with(uint32_t* chunk_hist, const uint32_t* indices, uint32_t* expert_counts,
                                    uint32_t* expert_offsets, uint32_t* expert_cursors, uint32_t* sorted_routes,
                                    uint32_t* sorted_experts, uint32_t* route_to_sorted, uint32_t routes, uint32_t experts,
                                    cudaStream_t stream) {
    const uint32_t chunks = (routes + kSortChunk - 1) / kSortChunk;
    moe_chunk_hist_kernel<<<chunks, kSortChunk, experts * sizeof(uint32_t), stream>>>(indices, chunk_hist, routes, experts);
    cudaError_t st = cudaGetLastError();
    if (st != cudaSuccess) return st;
    moe_prefix_kernel<<<1, 1024, 0, stream>>>(chunk_hist, expert_counts, expert_offsets, expert_cursors, chunks, experts);
    st = cudaGetLastError();
    if (st != cudaSuccess) return st;
    moe_scatter_kernel<<<chunks, kSortChunk, (kSortChunk / 32) * experts * sizeof(uint32_t), stream>>>(
        indices, chunk_hist, expert_offsets, sorted_routes, sorted_experts, route_to_sorted, routes, experts);
    return cudaGetLastError();
}

cudaError_t eider_b200_moe_sort_routes_on_stream(const uint32_t* indices, uint32_t* expert_counts, uint32_t* expert_offsets,
                                                 uint32_t* expert_cursors, uint32_t* sorted_routes, uint32_t* sorted_experts,
                                                 uint32_t* route_to_sorted, uint32_t routes, uint32_t experts, void* scratch,
                                                 size_t scratch_bytes, cudaStream_t stream) {
    if (!indices || !expert_counts || !expert_offsets || !expert_cursors || !sorted_routes || !sorted_experts ||
        !route_to_sorted || !scratch || routes == 0 || experts == 0 || experts > 1024 ||
        scratch_bytes < eider_b200_moe_sort_scratch_bytes(routes, experts))
        return cudaErrorInvalidValue;
    return sort_routes_with(static_cast<uint32_t*>(scratch), indices, expert_counts, expert_offsets, expert_cursors, sorted_routes,
                            sorted_experts, route_to_sorted, routes, experts, stream);
}

// Route sort for callers that cannot hand over scratch memory and must not trigger an allocation: same outputs as
// eider_b200_moe_sort_routes_on_stream, with the chunk histograms kept in a table that is part of the library image.
// The first call on a device looks up the table's device address (make that call outside any stream capture); every
// call shares the one table, so two sorts that overlap on the same GPU corrupt each other.  Nothing in the table has to
// be cleared between calls: each sort overwrites every entry it later reads.
cudaError_t eider_b200_moe_sort_routes_noalloc_on_stream(const uint32_t* indices, uint32_t* expert_counts,
                                                         uint32_t* expert_offsets, uint32_t* expert_cursors,
                                                         uint32_t* sorted_routes, uint32_t* sorted_experts,
                                                         uint32_t* route_to_sorted, uint32_t routes, uint32_t experts,
                                                         cudaStream_t stream) {
    if (!indices || !expert_counts || !expert_offsets || !expert_cursors || !sorted_routes || !sorted_experts ||
        !route_to_sorted || routes == 0 || experts == 0 || experts > 1024)
        return cudaErrorInvalidValue;
    const uint32_t chunks = (routes + kSortChunk - 1) / kSortChunk;
    if (static_cast<uint64_t>(chunks) * experts > kNoAllocSortEntries) return cudaErrorInvalidValue;  // beyond the built-in table
    uint32_t* chunk_hist = nullptr;
    cudaError_t st = noalloc_sort_scratch(&chunk_hist);
    if (st != cudaSuccess) return st;
    return sort_routes_with(chunk_hist, indices, expert_counts, expert_offsets, expert_cursors, sorted_routes, sorted_experts,
                            route_to_sorted, routes, experts, stream);
}

// crates/eider-cuda/src/ffi.rs:1701: the reference's sort call, which passes no scratch.  Same stable sort through the
// table inside the library, hence the same size limit and the same rule about overlapping calls as the entry point above.
cudaError_t infer_moe_sort_routes_on_stream(const uint32_t* indices, uint32_t* expert_counts, uint32_t* expert_offsets,
                                            uint32_t* expert_cursors, uint32_t* sorted_routes, uint32_t* sorted_experts,
                                            uint32_t* route_to_sorted, uint32_t routes, uint32_t experts, cudaStream_t stream) {
    return eider_b200_moe_sort_routes_noalloc_on_stream(indices, expert_counts, expert_offsets, expert_cursors, sorted_routes,
                                                        sorted_experts, route_to_sorted, routes, experts, stream);
}

size_t eider_b200_moe_sort_noalloc_max_entries(void) { return kNoAllocSortEntries; }

cudaError_t infer_moe_gather_quantize_sorted_routes_nvfp4_on_stream(const float* input, const uint32_t* sorted_routes,
                                                                    const uint32_t* sorted_experts,
                                                                    const uint32_t* expert_offsets, uint8_t* source_packed,
                                                                    uint8_t* source_scales, uint8_t* packed, uint8_t* scales,
                                                                    uint32_t rows, uint32_t routes, uint32_t routes_per_row,
                                                                    uint32_t in_features, uint32_t scale_tile_bytes,
                                                                    cudaStream_t stream) {
    if (!input || !sorted_routes || !sorted_experts || !expert_offsets || !source_packed || !source_scales || !packed ||
        !scales || rows == 0 || routes == 0 || routes_per_row == 0 || in_features == 0 || in_features % 16 != 0 ||
        scale_tile_bytes == 0)
        return cudaErrorInvalidValue;
    cudaError_t st = infer_quantize_nvfp4_col_major_f32_on_stream(input, source_packed, source_scales, in_features, rows, 1.0f,
                                                                  stream);
    if (st != cudaSuccess) return st;
    moe_scatter_rows_kernel<<<(routes + kScatterWarps - 1) / kScatterWarps, kScatterWarps * 32, 0, stream>>>(
        source_packed, source_scales, sorted_routes, sorted_experts, expert_offsets, packed, scales, routes, routes_per_row,
        in_features, scale_tile_bytes, 1);
    return cudaGetLastError();
}

cudaError_t eider_b200_moe_gather_quantize_sorted_routes_nvfp4_bf16_on_stream(
    const uint16_t* input, const uint32_t* sorted_routes, const uint32_t* sorted_experts, const uint32_t* expert_offsets,
    uint8_t* source_packed, uint8_t* source_scales, uint8_t* packed, uint8_t* scales, uint32_t rows, uint32_t routes,
    uint32_t routes_per_row, uint32_t in_features, uint32_t scale_tile_bytes, cudaStream_t stream) {
    if (!input || !sorted_routes || !sorted_experts || !expert_offsets || !source_packed || !source_scales || !packed ||
        !scales || rows == 0 || routes == 0 || routes_per_row == 0 || in_features == 0 || in_features % 16 != 0 ||
        scale_tile_bytes == 0)
        return cudaErrorInvalidValue;
    cudaError_t st = eider_b200_quantize_nvfp4_bf16_on_stream(input, source_packed, source_scales, in_features, rows, 1.0f, stream);
    if (st != cudaSuccess) return st;
    moe_scatter_rows_kernel<<<(routes + kScatterWarps - 1) / kScatterWarps, kScatterWarps * 32, 0, stream>>>(
        source_packed, source_scales, sorted_routes, sorted_experts, expert_offsets, packed, scales, routes, routes_per_row,
        in_features, scale_tile_bytes, 1);
    return cudaGetLastError();
}

cudaError_t eider_b200_moe_silu_mul_halves_quantize_sorted_routes_nvfp4_limited_on_stream(
    const uint16_t* gate_up, const uint32_t* sorted_experts, const uint32_t* expert_offsets, uint8_t* packed, uint8_t* scales,
    uint32_t routes, uint32_t in_features, uint32_t scale_tile_bytes, const uint32_t* routes_limit, cudaStream_t stream) {
    if (!gate_up || !sorted_experts || !expert_offsets || !packed || !scales || routes == 0 || in_features == 0 ||
        in_features % 16 != 0 || scale_tile_bytes == 0 || (reinterpret_cast<uintptr_t>(gate_up) & 15) != 0)
        return cudaErrorInvalidValue;
    const uint64_t units = static_cast<uint64_t>(routes) * (in_features / 8);
    moe_silu_mul_quantize_kernel<<<static_cast<uint32_t>((units + 255) / 256), 256, 0, stream>>>(
        gate_up, sorted_experts, expert_offsets, packed, scales, routes, in_features, scale_tile_bytes, routes_limit);
    return cudaGetLastError();
}

cudaError_t infer_moe_silu_mul_halves_quantize_sorted_routes_nvfp4_on_stream(const uint16_t* gate_up,
                                                                             const uint32_t* sorted_experts,
                                                                             const uint32_t* expert_offsets, uint8_t* packed,
                                                                             uint8_t* scales, uint32_t routes,
                                                                             uint32_t in_features, uint32_t scale_tile_bytes,
                                                                             cudaStream_t stream) {
    return eider_b200_moe_silu_mul_halves_quantize_sorted_routes_nvfp4_limited_on_stream(
        gate_up, sorted_experts, expert_offsets, packed, scales, routes, in_features, scale_tile_bytes, nullptr, stream);
}

static cudaError_t launch_sorted_quant(int mode, const void* input, const void* input2, const float* input_scales,
                                       const uint32_t* sorted_routes, const uint32_t* sorted_experts,
                                       const uint32_t* expert_offsets, uint8_t* packed, uint8_t* scales, uint32_t routes,
                                       uint32_t routes_per_row, uint32_t k, uint32_t tile_bytes, int gather_rows,
                                       cudaStream_t stream) {
    if (!input || !sorted_routes || !sorted_experts || !expert_offsets || !packed || !scales || routes == 0 ||
        routes_per_row == 0 || k == 0 || k % 16 != 0 || tile_bytes == 0 || (reinterpret_cast<uintptr_t>(packed) & 7) != 0)
        return cudaErrorInvalidValue;
    const uint64_t units = static_cast<uint64_t>(routes) * (k / 16);
    const uint32_t grid = static_cast<uint32_t>((units + 255) / 256);
#define EIDER_SORTED_QUANT(M)                                                                                                  \
    moe_quantize_sorted_kernel<M><<<grid, 256, 0, stream>>>(input, input2, input_scales, sorted_routes, sorted_experts,        \
                                                            expert_offsets, packed, scales, routes, routes_per_row, k, tile_bytes, \
                                                            gather_rows)
    switch (mode) {
        case kPlain: EIDER_SORTED_QUANT(kPlain); break;
        case kCalibrated: EIDER_SORTED_QUANT(kCalibrated); break;
        case kReluSquared: EIDER_SORTED_QUANT(kReluSquared); break;
        default: EIDER_SORTED_QUANT(kGeluPair); break;
    }
#undef EIDER_SORTED_QUANT
    return cudaGetLastError();
}

cudaError_t infer_moe_quantize_sorted_routes_nvfp4_on_stream(const float* input, const uint32_t* sorted_routes,
                                                             const uint32_t* sorted_experts, const uint32_t* expert_offsets,
                                                             uint8_t* packed, uint8_t* scales, uint32_t routes,
                                                             uint32_t routes_per_row, uint32_t in_features,
                                                             uint32_t scale_tile_bytes, int gather_rows, cudaStream_t stream) {
    return launch_sorted_quant(kPlain, input, nullptr, nullptr, sorted_routes, sorted_experts, expert_offsets, packed, scales,
                               routes, routes_per_row, in_features, scale_tile_bytes, gather_rows, stream);
}

cudaError_t infer_moe_calibrated_quantize_on_stream(const void* input, const float* input_scales, const uint32_t* sorted_routes,
                                                    const uint32_t* sorted_experts, const uint32_t* expert_offsets,
                                                    uint8_t* packed, uint8_t* scales, uint32_t routes, uint32_t routes_per_row,
                                                    uint32_t features, uint32_t scale_tile_bytes, int relu_squared,
                                                    cudaStream_t stream) {
    if (!input_scales) return cudaErrorInvalidValue;
    return launch_sorted_quant(relu_squared ? kReluSquared : kCalibrated, input, nullptr, input_scales, sorted_routes,
                               sorted_experts, expert_offsets, packed, scales, routes, routes_per_row, features,
                               scale_tile_bytes, 1, stream);
}

cudaError_t infer_moe_gelu_tanh_mul_quantize_sorted_routes_nvfp4_on_stream(const uint16_t* gate, const uint16_t* up,
                                                                           const uint32_t* sorted_experts,
                                                                           const uint32_t* expert_offsets, uint8_t* packed,
                                                                           uint8_t* scales, uint32_t routes, uint32_t in_features,
                                                                           uint32_t scale_tile_bytes, cudaStream_t stream) {
    if (!up) return cudaErrorInvalidValue;
    // (the kernel reads no route ids in this mode; the expert ids stand in for the non-null argument)
    return launch_sorted_quant(kGeluPair, gate, up, nullptr, sorted_experts, sorted_experts, expert_offsets, packed, scales, routes,
                               1, in_features, scale_tile_bytes, 0, stream);
}

cudaError_t infer_moe_gather_rms_norm_quantize_sorted_routes_nvfp4_on_stream(
    const float* input, const float* weight, const uint32_t* sorted_routes, const uint32_t* sorted_experts,
    const uint32_t* expert_offsets, uint8_t* source_packed, uint8_t* source_scales, uint8_t* packed, uint8_t* scales,
    uint32_t rows, uint32_t routes, uint32_t routes_per_row, uint32_t in_features, uint32_t scale_tile_bytes, float eps,
    cudaStream_t stream) {
    if (!input || !weight || !sorted_routes || !sorted_experts || !expert_offsets || !source_packed || !source_scales ||
        !packed || !scales || rows == 0 || routes == 0 || routes_per_row == 0 || in_features == 0 || in_features % 16 != 0 ||
        scale_tile_bytes == 0)
        return cudaErrorInvalidValue;
    // every token is normalised and quantized once (unit global scale), then its bytes are scattered to its routes
    cudaError_t st = infer_rms_norm_quantize_nvfp4_col_major_f32_on_stream(input, weight, source_packed, source_scales, rows,
                                                                           in_features, eps, 1.0f, stream);
    if (st != cudaSuccess) return st;
    moe_scatter_rows_kernel<<<(routes + kScatterWarps - 1) / kScatterWarps, kScatterWarps * 32, 0, stream>>>(
        source_packed, source_scales, sorted_routes, sorted_experts, expert_offsets, packed, scales, routes, routes_per_row,
        in_features, scale_tile_bytes, 1);
    return cudaGetLastError();
}

cudaError_t infer_moe_grouped_pointer_tables_on_stream(const uint32_t* expert_offsets, const uint8_t* packed,
                                                       const uint8_t* scales, uint16_t* output, const uint8_t** packed_table,
                                                       const uint8_t** scale_table, uint16_t** output_table, uint32_t experts,
                                                       uint32_t in_features, uint32_t out_features, uint32_t scale_tile_bytes,
                                                       cudaStream_t stream) {
    if (!expert_offsets || !packed || !scales || !output || !packed_table || !scale_table || !output_table || experts == 0 ||
        in_features == 0 || out_features == 0 || scale_tile_bytes == 0)
        return cudaErrorInvalidValue;
    moe_pointer_tables_kernel<<<(experts + 127) / 128, 128, 0, stream>>>(expert_offsets, packed, scales, output, packed_table,
                                                                        scale_table, output_table, experts, in_features,
                                                                        out_features, scale_tile_bytes);
    return cudaGetLastError();
}

cudaError_t infer_moe_weighted_accumulate_sorted_bf16_batch_on_stream(const uint32_t* route_to_sorted,
                                                                      const float* route_weights,
                                                                      const uint16_t* sorted_inputs, float* output,
                                                                      uint32_t rows, uint32_t len, uint32_t routes_per_row,
                                                                      cudaStream_t stream) {
    if (!route_to_sorted || !route_weights || !sorted_inputs || !output || rows == 0 || len == 0 || routes_per_row == 0)
        return cudaErrorInvalidValue;
    const bool vec = len % 8 == 0 && (reinterpret_cast<uintptr_t>(sorted_inputs) & 15) == 0 &&
                     (reinterpret_cast<uintptr_t>(output) & 15) == 0;
    if (vec) {
        const size_t total = static_cast<size_t>(rows) * (len / 8);
        moe_combine_kernel<<<static_cast<uint32_t>((total + 255) / 256), 256, 0, stream>>>(route_to_sorted, route_weights,
                                                                                         sorted_inputs, output, rows, len,
                                                                                         routes_per_row);
    } else {
        const size_t total = static_cast<size_t>(rows) * len;
        moe_combine_scalar_kernel<<<static_cast<uint32_t>((total + 255) / 256), 256, 0, stream>>>(
            route_to_sorted, route_weights, sorted_inputs, output, rows, len, routes_per_row);
    }
    return cudaGetLastError();
}

}  // extern "C"
