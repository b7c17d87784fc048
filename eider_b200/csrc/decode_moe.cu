// Decode-side routed MoE (one to a few tokens, top-k slots each): grouped GEMVs over per-expert weight tables, the
// per-slot SiLU * up stage, the weighted accumulation of the slots and the shared-expert / residual finalize, plus the
// fused lm-head GEMV + arg-max.  Everything a decode step of the reference's routed layers calls between the router and
// the residual stream (crates/eider-cuda/native/non_gemm.cu:3396-3960, 13316-13640; crates/eider-cuda/native/
// cutlass_gemv.cu:277-880), under the reference's names.
//
// All of it is HBM-bound streaming: a slot's expert matrix is read exactly once with 128-bit loads, one warp per output
// row, activations staged once per CTA in shared memory, warp-shuffle reduction; the experts of the slots are found
// through device pointer tables, so nothing is gathered or copied first.  Products are exact in f32 (an E2M1 value times
// an f32 activation, or times another E2M1 value) and only the order of the additions differs from the reference.
#include "common.cuh"
#include "eider_b200.h"

namespace eider {
namespace {

constexpr int kWarps = 8;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Shared-memory slot of element e (0..31) of 32-element chunk c: float4 slots XOR-swizzled by the chunk so that lanes
// reading the same slot of consecutive chunks hit distinct banks.
__device__ __forceinline__ uint32_t xs_index(uint32_t c, uint32_t e) { return c * 32 + ((((e >> 2) ^ (c & 7u)) << 2) | (e & 3u)); }

__device__ __forceinline__ void dot_word(uint32_t w, const float* xs, uint32_t c, uint32_t e0, float& acc) {
    const float4 a = *reinterpret_cast<const float4*>(xs + xs_index(c, e0));
    const float4 b = *reinterpret_cast<const float4*>(xs + xs_index(c, e0 + 4));
    acc = fmaf(e2m1_value(w), a.x, acc);
    acc = fmaf(e2m1_value(w >> 4), a.y, acc);
    acc = fmaf(e2m1_value(w >> 8), a.z, acc);
    acc = fmaf(e2m1_value(w >> 12), a.w, acc);
    acc = fmaf(e2m1_value(w >> 16), b.x, acc);
    acc = fmaf(e2m1_value(w >> 20), b.y, acc);
    acc = fmaf(e2m1_value(w >> 24), b.z, acc);
    acc = fmaf(e2m1_value(w >> 28), b.w, acc);
}

enum XMode { kSharedF32 = 0, kTableF32 = 1, kSharedNvfp4 = 2 };

struct GroupedArgs {
    const uint32_t* indices;          // [groups] expert of every slot (null: slot g uses table entry g)
    const void* x;                    // kSharedF32: f32 [k]; kTableF32: const float* const* [groups]; kSharedNvfp4: packed [k/2]
    const uint8_t* x_scales;          // kSharedNvfp4: tiled scales of the one activation row (outer = 0)
    const uint8_t* const* w_table;    // [table_len] packed weights [n][k/2]
    const uint8_t* const* s_table;    // [table_len] weight scales: row-major [n][k/16] or tiled (TILED)
    const float* alpha_table;         // [table_len] per-expert factor (null: alpha)
    float alpha;
    float* const* y_table;            // [groups] outputs [n] (null: y_flat + g * n)
    float* y_flat;
    uint32_t table_len, groups, n, k;
    const uint32_t* route_ids = nullptr;  // kTableF32: when set, slot g reads input (and writes output) route_ids[g] of the tables
};

// grid = (ceil(n / kWarps), groups); k % 32 == 0.
template <int XMODE, bool TILED>
__global__ void __launch_bounds__(kWarps * 32) grouped_gemv_kernel(const GroupedArgs a) {
    extern __shared__ float xs[];  // [k], swizzled
    const uint32_t group = blockIdx.y;
    const uint32_t expert = a.indices ? __ldg(a.indices + group) : group;
    if (expert >= a.table_len) return;  // (the reference skips such slots, non_gemm.cu:13342-13345)
    const uint32_t k = a.k;
    if (XMODE == kSharedNvfp4) {
        const uint8_t* xp = static_cast<const uint8_t*>(a.x);
        for (uint32_t i = threadIdx.x; i < k / 2; i += blockDim.x) {
            const uint32_t byte = __ldg(xp + i);
            const float s = e4m3_value(__ldg(a.x_scales + tiled_scale_offset(0, i / 8, k)));
            const uint32_t e = 2 * i;
            xs[xs_index(e / 32, e % 32)] = __fmul_rn(e2m1_value(byte), s);
            xs[xs_index(e / 32, e % 32 + 1)] = __fmul_rn(e2m1_value(byte >> 4), s);
        }
    } else {
        const uint32_t x_slot = (XMODE == kTableF32 && a.route_ids) ? __ldg(a.route_ids + group) : group;
        const float* x = XMODE == kTableF32 ? static_cast<const float* const*>(a.x)[x_slot] : static_cast<const float*>(a.x);
        for (uint32_t i = threadIdx.x; i < k; i += blockDim.x) xs[xs_index(i / 32, i % 32)] = __ldg(x + i);
    }
    __syncthreads();
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t row = blockIdx.x * kWarps + (threadIdx.x >> 5);
    if (row >= a.n) return;
    const uint8_t* wrow = a.w_table[expert] + static_cast<size_t>(row) * (k / 2);
    const uint8_t* sbase = a.s_table[expert];
    float acc = 0.0f;
    for (uint32_t c = lane; c < k / 32; c += 32) {
        const uint4 q = __ldg(reinterpret_cast<const uint4*>(wrow + c * 16));
        uint32_t sc;
        if (TILED) sc = __ldg(reinterpret_cast<const uint16_t*>(sbase + tiled_scale_offset(row, c * 2, k)));  // blocks 2c, 2c + 1 are adjacent
        else sc = __ldg(reinterpret_cast<const uint16_t*>(sbase + static_cast<size_t>(row) * (k / 16) + c * 2));
        float p0 = 0.0f, p1 = 0.0f;
        dot_word(q.x, xs, c, 0, p0);
        dot_word(q.y, xs, c, 8, p0);
        dot_word(q.z, xs, c, 16, p1);
        dot_word(q.w, xs, c, 24, p1);
        acc = fmaf(e4m3_value(static_cast<uint8_t>(sc & 0xff)), p0, acc);
        acc = fmaf(e4m3_value(static_cast<uint8_t>(sc >> 8)), p1, acc);
    }
    acc = warp_sum(acc);
    if (lane == 0) {
        const uint32_t y_slot = (XMODE == kTableF32 && a.route_ids) ? __ldg(a.route_ids + group) : group;
        float* y = a.y_table ? a.y_table[y_slot] : a.y_flat + static_cast<size_t>(y_slot) * a.n;
        y[row] = __fmul_rn(acc, a.alpha_table ? __ldg(a.alpha_table + expert) : a.alpha);
    }
}

template <int XMODE, bool TILED>
cudaError_t launch_grouped(const GroupedArgs& a, cudaStream_t stream) {
    if (a.k == 0 || a.k % 32 != 0 || a.n == 0 || a.groups == 0 || a.table_len == 0) return cudaErrorInvalidValue;
    const size_t smem = static_cast<size_t>(a.k) * sizeof(float);
    if (smem > 200 * 1024) return cudaErrorNotSupported;
    if (smem > 48 * 1024) {
        cudaError_t st = cudaFuncSetAttribute(grouped_gemv_kernel<XMODE, TILED>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        if (st != cudaSuccess) return st;
    }
    const dim3 grid((a.n + kWarps - 1) / kWarps, a.groups);
    grouped_gemv_kernel<XMODE, TILED><<<grid, kWarps * 32, smem, stream>>>(a);
    return cudaGetLastError();
}

// gate * alpha, up * alpha, then gate * sigmoid(gate) * up (non_gemm.cu:3507-3511, 3570-3574)
__device__ __forceinline__ float slot_silu(float g, float u, float alpha) {
    g = __fmul_rn(g, alpha);
    u = __fmul_rn(u, alpha);
    const float sigmoid = __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-g)));
    return __fmul_rn(__fmul_rn(g, sigmoid), u);
}

// Per slot: SiLU(gate) * up of the slot's [gate | up] f32 row -> f32 (non_gemm.cu:3558-3576).  grid = (blocks, groups).
__global__ void __launch_bounds__(256) silu_slots_f32_kernel(const uint32_t* __restrict__ indices, const float* const* gate_up_table,
                                                             float* const* output_table, const float* __restrict__ alpha_table,
                                                             uint32_t rows) {
    const uint32_t slot = blockIdx.y;
    const uint32_t row = blockIdx.x * blockDim.x + threadIdx.x;
    if (row >= rows) return;
    const float alpha = __ldg(alpha_table + __ldg(indices + slot));
    const float* gu = gate_up_table[slot];
    output_table[slot][row] = slot_silu(__ldg(gu + row), __ldg(gu + rows + row), alpha);
}

// Per slot: the same values / input_scale[expert] -> NVFP4 with one scale byte per 16 values in plain order
// (non_gemm.cu:3485-3536).  One thread per 16-value block; grid = (blocks of 128 threads, groups).
__global__ void __launch_bounds__(128) silu_quantize_slots_kernel(const uint32_t* __restrict__ indices, const float* const* gate_up_table,
                                                                  uint8_t* const* packed_table, uint8_t* const* scales_table,
                                                                  const float* __restrict__ input_scale_table,
                                                                  const float* __restrict__ alpha_table, uint32_t rows) {
    const uint32_t slot = blockIdx.y;
    const uint32_t b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= (rows + 15) / 16) return;
    const uint32_t expert = __ldg(indices + slot);
    const float input_scale = __ldg(input_scale_table + expert);
    if (!(input_scale > 0.0f) || !isfinite(input_scale)) return;  // (as the reference: such a slot is left untouched)
    const float alpha = __ldg(alpha_table + expert);
    const float* gu = gate_up_table[slot];
    const uint32_t valid = min(16u, rows - b * 16);
    const Divisor di = make_divisor(input_scale);
    float v[16];
#pragma unroll
    for (int i = 0; i < 16; ++i)
        v[i] = static_cast<uint32_t>(i) < valid ? div_rn(slot_silu(__ldg(gu + b * 16 + i), __ldg(gu + rows + b * 16 + i), alpha), di) : 0.0f;
    uint2 bytes;
    scales_table[slot][b] = quantize_block16(v, valid, &bytes);
    const uint32_t w[2] = {bytes.x, bytes.y};
    uint8_t* packed = packed_table[slot];
    for (uint32_t i = 0; i < (valid + 1) / 2; ++i) packed[b * 8 + i] = static_cast<uint8_t>(w[i / 4] >> ((i % 4) * 8));
}

// out[row][c] = sum_slot inputs[route][c] * route_weights[route] * alpha[expert(route)], slot order (non_gemm.cu:3595-3639);
// with FINALIZE: + shared_output * sigmoid(shared_gate_logit) + residual, rounded to bf16 precision (non_gemm.cu:3789-3875).
template <bool FINALIZE>
__global__ void __launch_bounds__(256) accumulate_slots_kernel(const uint32_t* __restrict__ indices, const float* __restrict__ route_weights,
                                                               const float* const* inputs, const float* __restrict__ alpha_table,
                                                               const float* __restrict__ shared_gate_logit,
                                                               const float* __restrict__ shared_output, const float* __restrict__ residual,
                                                               float* __restrict__ output, uint32_t rows, uint32_t len, uint32_t groups) {
    const size_t idx = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= static_cast<size_t>(rows) * len) return;
    const uint32_t row = static_cast<uint32_t>(idx / len), col = static_cast<uint32_t>(idx % len);
    float sum = 0.0f;
    for (uint32_t slot = 0; slot < groups; ++slot) {
        const uint32_t route = row * groups + slot;
        // inputs * weight * alpha + sum, the last two as one fused multiply-add (what nvcc makes of non_gemm.cu:3609)
        sum = fmaf(__fmul_rn(inputs[route][col], __ldg(route_weights + route)), __ldg(alpha_table + __ldg(indices + route)), sum);
    }
    if (FINALIZE) {
        const float shared_scale = __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-__ldg(shared_gate_logit + row))));
        const float ffn = __fadd_rn(sum, __fmul_rn(__ldg(shared_output + idx), shared_scale));
        sum = bf16_bits_to_float(float_to_bf16_bits(__fadd_rn(__ldg(residual + idx), ffn)));
    }
    output[idx] = sum;
}

// Fused lm-head GEMV + arg-max (non_gemm.cu:13423-13640): pass 1 keeps, per CTA, the best (value, row) of its rows; pass 2
// reduces the per-CTA candidates.  The logits are never written.  Ties go to the lower row, NaN never wins.
__global__ void __launch_bounds__(kWarps * 32) top1_pass1_kernel(const float* __restrict__ x, const uint8_t* __restrict__ w,
                                                                 const uint8_t* __restrict__ s, float w2, uint32_t n, uint32_t k,
                                                                 float* __restrict__ block_value, uint32_t* __restrict__ block_row) {
    extern __shared__ float xs[];
    __shared__ float best_v[kWarps];
    __shared__ uint32_t best_r[kWarps];
    for (uint32_t i = threadIdx.x; i < k; i += blockDim.x) xs[xs_index(i / 32, i % 32)] = __ldg(x + i);
    __syncthreads();
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    // every warp walks rows warp, warp + kWarps * gridDim.x ... of this CTA's share
    float bv = -INFINITY;
    uint32_t br = 0xffffffffu;
    for (uint32_t row = blockIdx.x * kWarps + warp; row < n; row += gridDim.x * kWarps) {
        const uint8_t* wrow = w + static_cast<size_t>(row) * (k / 2);
        const uint8_t* srow = s + static_cast<size_t>(row) * (k / 16);
        float acc = 0.0f;
        for (uint32_t c = lane; c < k / 32; c += 32) {
            const uint4 q = __ldg(reinterpret_cast<const uint4*>(wrow + c * 16));
            const uint32_t sc = __ldg(reinterpret_cast<const uint16_t*>(srow + c * 2));
            float p0 = 0.0f, p1 = 0.0f;
            dot_word(q.x, xs, c, 0, p0);
            dot_word(q.y, xs, c, 8, p0);
            dot_word(q.z, xs, c, 16, p1);
            dot_word(q.w, xs, c, 24, p1);
            acc = fmaf(e4m3_value(static_cast<uint8_t>(sc & 0xff)), p0, acc);
            acc = fmaf(e4m3_value(static_cast<uint8_t>(sc >> 8)), p1, acc);
        }
        const float v = __fmul_rn(warp_sum(acc), w2);
        if (v > bv || (v == bv && row < br)) {
            bv = v;
            br = row;
        }
    }
    if (lane == 0) {
        best_v[warp] = bv;
        best_r[warp] = br;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int i = 1; i < kWarps; ++i)
            if (best_v[i] > bv || (best_v[i] == bv && best_r[i] < br)) {
                bv = best_v[i];
                br = best_r[i];
            }
        block_value[blockIdx.x] = bv;
        block_row[blockIdx.x] = br;
    }
}

__global__ void __launch_bounds__(256) top1_pass2_kernel(const float* __restrict__ block_value, const uint32_t* __restrict__ block_row,
                                                         uint32_t blocks, uint32_t* __restrict__ out_index, float* __restrict__ out_value) {
    __shared__ float sv[256];
    __shared__ uint32_t sr[256];
    float bv = -INFINITY;
    uint32_t br = 0xffffffffu;
    for (uint32_t i = threadIdx.x; i < blocks; i += blockDim.x) {
        const float v = block_value[i];
        const uint32_t r = block_row[i];
        if (v > bv || (v == bv && r < br)) {
            bv = v;
            br = r;
        }
    }
    sv[threadIdx.x] = bv;
    sr[threadIdx.x] = br;
    __syncthreads();
    for (uint32_t o = 128; o > 0; o >>= 1) {
        if (threadIdx.x < o) {
            const float v = sv[threadIdx.x + o];
            const uint32_t r = sr[threadIdx.x + o];
            if (v > sv[threadIdx.x] || (v == sv[threadIdx.x] && r < sr[threadIdx.x])) {
                sv[threadIdx.x] = v;
                sr[threadIdx.x] = r;
            }
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        out_index[0] = sr[0] == 0xffffffffu ? 0u : sr[0];  // (all rows NaN: row 0, as an arg-max over nothing better)
        if (out_value) out_value[0] = sv[0];
    }
}

// ---- FP8 W8A8 slots (crates/eider-cuda/native/non_gemm.cu:10156-10350) ------------------------------------------------------
// One warp per output row, the slot's activation codes decoded once per CTA into shared memory, weights streamed with 128-bit
// loads; every product of two E4M3 values is exact in f32.  GATE_UP: rows [0, n) come from the gate table and [n, 2n) from
// the up table, one shared activation; otherwise one activation row per slot and one output vector per slot.
template <bool GATE_UP>
__global__ void __launch_bounds__(kWarps * 32) fp8_slot_gemv_kernel(const uint32_t* __restrict__ indices, const uint8_t* __restrict__ x_codes,
                                                                    const float* __restrict__ x_scales, const uint8_t* const* w_table,
                                                                    const float* const* s_table, const uint8_t* const* w2_table,
                                                                    const float* const* s2_table, float* y_flat, float* const* y_table,
                                                                    uint32_t n, uint32_t k) {
    extern __shared__ float xs[];  // [k], swizzled
    const uint32_t slot = blockIdx.y;
    const uint32_t expert = __ldg(indices + slot);
    const uint8_t* x = GATE_UP ? x_codes : x_codes + static_cast<size_t>(slot) * k;
    for (uint32_t i = threadIdx.x; i < k; i += blockDim.x) xs[xs_index(i / 32, i % 32)] = e4m3_value(__ldg(x + i));
    __syncthreads();
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t row = blockIdx.x * kWarps + (threadIdx.x >> 5);
    const uint32_t total = GATE_UP ? 2 * n : n;
    if (row >= total) return;
    const bool second = GATE_UP && row >= n;
    const uint32_t r = second ? row - n : row;
    const uint8_t* wrow = (second ? w2_table[expert] : w_table[expert]) + static_cast<size_t>(r) * k;
    float acc = 0.0f;
    for (uint32_t h = lane; h < k / 16; h += 32) {
        const uint4 q = __ldg(reinterpret_cast<const uint4*>(wrow + h * 16));
        const uint32_t ww[4] = {q.x, q.y, q.z, q.w};
        const uint32_t c = h / 2, e0 = (h & 1) * 16;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float4 a = *reinterpret_cast<const float4*>(xs + xs_index(c, e0 + 4 * j));
            acc = fmaf(e4m3_value(static_cast<uint8_t>(ww[j])), a.x, acc);
            acc = fmaf(e4m3_value(static_cast<uint8_t>(ww[j] >> 8)), a.y, acc);
            acc = fmaf(e4m3_value(static_cast<uint8_t>(ww[j] >> 16)), a.z, acc);
            acc = fmaf(e4m3_value(static_cast<uint8_t>(ww[j] >> 24)), a.w, acc);
        }
    }
    acc = warp_sum(acc);
    if (lane == 0) {
        const float sx = GATE_UP ? __ldg(x_scales) : __ldg(x_scales + slot);
        const float sw = __ldg((second ? s2_table[expert] : s_table[expert]) + r);
        const float v = __fmul_rn(__fmul_rn(acc, sx), sw);
        if (GATE_UP) y_flat[static_cast<size_t>(slot) * 2 * n + row] = v;
        else y_table[slot][row] = v;
    }
}

// Per slot: SiLU(gate) * up of the slot's [gate | up] row, one dynamic scale amax / 448 per slot (1 for an all-zero slot;
// non-finite values do not enter the maximum), E4M3 codes (non_gemm.cu:10241-10270).  One CTA per slot.
__global__ void __launch_bounds__(256) silu_quantize_fp8_slots_kernel(const float* __restrict__ gate_up, uint8_t* __restrict__ quantized,
                                                                      float* __restrict__ scales, uint32_t rows) {
    __shared__ float red[8];
    __shared__ float scale_sh;
    const uint32_t slot = blockIdx.x;
    const float* gate = gate_up + static_cast<size_t>(slot) * rows * 2;
    const float* up = gate + rows;
    float amax = 0.0f;
    for (uint32_t i = threadIdx.x; i < rows; i += 256) {
        const float g = __ldg(gate + i);
        const float v = __fmul_rn(__fdiv_rn(g, __fadd_rn(1.0f, expf(-g))), __ldg(up + i));
        if (isfinite(v)) amax = fmaxf(amax, fabsf(v));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int i = 1; i < 8; ++i) amax = fmaxf(amax, red[i]);
        const float sc = amax == 0.0f ? 1.0f : __fdiv_rn(amax, 448.0f);
        scales[slot] = sc;
        scale_sh = sc;
    }
    __syncthreads();
    const float sc = scale_sh;
    for (uint32_t i = threadIdx.x; i < rows; i += 256) {
        const float g = __ldg(gate + i);
        const float v = __fmul_rn(__fdiv_rn(g, __fadd_rn(1.0f, expf(-g))), __ldg(up + i));
        quantized[static_cast<size_t>(slot) * rows + i] = e4m3_satfinite(__fdiv_rn(v, sc));
    }
}

template <bool GATE_UP>
cudaError_t launch_fp8_slots(const uint32_t* indices, const uint8_t* x, const float* x_scales, const uint8_t* const* w, const float* const* s,
                             const uint8_t* const* w2, const float* const* s2, float* y_flat, float* const* y_table, uint32_t n, uint32_t k,
                             uint32_t slots, cudaStream_t stream) {
    if (k % 16 != 0) return cudaErrorInvalidValue;
    const size_t smem = static_cast<size_t>((k + 31) / 32 * 32) * sizeof(float);
    if (smem > 200 * 1024) return cudaErrorNotSupported;
    if (smem > 48 * 1024) {
        cudaError_t st = cudaFuncSetAttribute(fp8_slot_gemv_kernel<GATE_UP>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        if (st != cudaSuccess) return st;
    }
    const uint32_t total = GATE_UP ? 2 * n : n;
    fp8_slot_gemv_kernel<GATE_UP><<<dim3((total + kWarps - 1) / kWarps, slots), kWarps * 32, smem, stream>>>(indices, x, x_scales, w, s, w2, s2,
                                                                                                              y_flat, y_table, n, k);
    return cudaGetLastError();
}

}  // namespace
}  // namespace eider

using namespace eider;

extern "C" {

// ---- FP8 W8A8 decode-side MoE slots (crates/eider-cuda/src/ffi.rs:3163-3196) ----------------------------------------------
cudaError_t infer_fp8_moe_grouped_gate_up_f32_on_stream(const uint32_t* indices, const uint8_t* input, const float* input_scale,
                                                        const uint8_t* const* gate_weights, const float* const* gate_scales,
                                                        const uint8_t* const* up_weights, const float* const* up_scales, float* output,
                                                        uint32_t rows, uint32_t cols, uint32_t slots, cudaStream_t stream) {
    if (!indices || !input || !input_scale || !gate_weights || !gate_scales || !up_weights || !up_scales || !output || rows == 0 ||
        cols == 0 || slots == 0)
        return cudaErrorInvalidValue;
    return launch_fp8_slots<true>(indices, input, input_scale, gate_weights, gate_scales, up_weights, up_scales, output, nullptr, rows, cols,
                                  slots, stream);
}

cudaError_t infer_moe_silu_quantize_fp8_slots_f32_on_stream(const float* gate_up, uint8_t* quantized, float* scales, uint32_t rows,
                                                            uint32_t slots, cudaStream_t stream) {
    if (!gate_up || !quantized || !scales || rows == 0 || slots == 0) return cudaErrorInvalidValue;
    silu_quantize_fp8_slots_kernel<<<slots, 256, 0, stream>>>(gate_up, quantized, scales, rows);
    return cudaGetLastError();
}

cudaError_t infer_fp8_moe_grouped_down_f32_on_stream(const uint32_t* indices, const uint8_t* inputs, const float* input_scales,
                                                     const uint8_t* const* weights, const float* const* weight_scales,
                                                     float* const* outputs, uint32_t rows, uint32_t cols, uint32_t slots,
                                                     cudaStream_t stream) {
    if (!indices || !inputs || !input_scales || !weights || !weight_scales || !outputs || rows == 0 || cols == 0 || slots == 0)
        return cudaErrorInvalidValue;
    return launch_fp8_slots<false>(indices, inputs, input_scales, weights, weight_scales, nullptr, nullptr, nullptr, outputs, rows, cols,
                                   slots, stream);
}


cudaError_t infer_nvfp4_w4a16_grouped_matvec_f32_on_stream(const uint32_t* indices, const float* input,
                                                           const uint8_t* const* packed_weight_table,
                                                           const uint8_t* const* weight_scale_table,
                                                           const float* weight_scale_2_table, float* const* output_table,
                                                           uint32_t table_len, uint32_t groups, uint32_t out_features,
                                                           uint32_t in_features, cudaStream_t stream) {
    if (!indices || !input || !packed_weight_table || !weight_scale_table || !weight_scale_2_table || !output_table)
        return cudaErrorInvalidValue;
    GroupedArgs a{indices, input, nullptr, packed_weight_table, weight_scale_table, weight_scale_2_table, 1.0f, output_table, nullptr,
                  table_len, groups, out_features, in_features};
    return launch_grouped<kSharedF32, false>(a, stream);
}

cudaError_t infer_nvfp4_w4a16_grouped_inputs_matvec_f32_on_stream(const uint32_t* indices, const float* const* input_table,
                                                                  const uint8_t* const* packed_weight_table,
                                                                  const uint8_t* const* weight_scale_table,
                                                                  const float* weight_scale_2_table, float* const* output_table,
                                                                  uint32_t table_len, uint32_t groups, uint32_t out_features,
                                                                  uint32_t in_features, cudaStream_t stream) {
    if (!indices || !input_table || !packed_weight_table || !weight_scale_table || !weight_scale_2_table || !output_table)
        return cudaErrorInvalidValue;
    GroupedArgs a{indices, input_table, nullptr, packed_weight_table, weight_scale_table, weight_scale_2_table, 1.0f, output_table,
                  nullptr, table_len, groups, out_features, in_features};
    return launch_grouped<kTableF32, false>(a, stream);
}

// crates/eider-cuda/src/ffi.rs:3333 (kernel non_gemm.cu:13640-13724): routes sorted by expert, every route with its own input
// and output vector found through the tables by its route id.  The reference shares each decoded weight among four routes
// of one expert; here every route's rows stream its expert's matrix with 128-bit loads (consecutive routes of one expert
// find it in L2), the products are the same exact f32 products and only the order of the additions differs.  `offsets` is
// required non-null as in the reference and is not read.
cudaError_t infer_nvfp4_w4a16_reuse_matvec_f32_on_stream(const uint32_t* sorted_routes, const uint32_t* sorted_experts,
                                                         const uint32_t* offsets, const float* const* inputs,
                                                         const uint8_t* const* weights, const uint8_t* const* scales,
                                                         const float* globals, float* const* outputs, uint32_t routes,
                                                         uint32_t experts, uint32_t out_features, uint32_t in_features,
                                                         cudaStream_t stream) {
    if (!sorted_routes || !sorted_experts || !offsets || !inputs || !weights || !scales || !globals || !outputs)
        return cudaErrorInvalidValue;
    GroupedArgs a{sorted_experts, inputs, nullptr, weights, scales, globals, 1.0f, outputs, nullptr, experts, routes, out_features, in_features};
    a.route_ids = sorted_routes;
    return launch_grouped<kTableF32, false>(a, stream);
}

// ---- W4A4 grouped GEMV (crates/eider-cuda/src/ffi.rs:589-642; crates/eider-cuda/native/cutlass_gemv.cu:277-880) ----------
// The plan only records the shape (the reference's holds CUTLASS workspace); it owns no device memory.
struct GroupedGemvPlan {
    uint32_t m, k, groups;
};

int infer_cutlass_fp4_grouped_gemv_f32_supported(uint32_t m, uint32_t k, uint32_t groups) {
    return (m > 0 && k > 0 && groups > 0 && k % 32 == 0 && static_cast<size_t>(k) * 4 <= 200 * 1024) ? 1 : 0;
}

void* infer_cutlass_fp4_grouped_gemv_f32_create(uint32_t m, uint32_t k, uint32_t groups) {
    if (!infer_cutlass_fp4_grouped_gemv_f32_supported(m, k, groups)) return nullptr;
    return new GroupedGemvPlan{m, k, groups};
}

void infer_cutlass_fp4_grouped_gemv_f32_destroy(void* plan) { delete static_cast<GroupedGemvPlan*>(plan); }

cudaError_t infer_cutlass_fp4_grouped_gemv_f32_indexed_a_tiled_scales_on_stream(void* raw, const uint32_t* indices,
                                                                                const uint8_t* const* a_values_table,
                                                                                const uint8_t* const* a_scales_table,
                                                                                const float* alpha_table, uint32_t table_len,
                                                                                const uint8_t* b_values, const uint8_t* b_scales,
                                                                                const float* c, float* const* d, cudaStream_t stream) {
    auto* plan = static_cast<GroupedGemvPlan*>(raw);
    (void)c;  // beta is 0 in the reference's call (cutlass_gemv.cu:640-648)
    if (!plan || !indices || !a_values_table || !a_scales_table || !alpha_table || !b_values || !b_scales || !d) return cudaErrorInvalidValue;
    GroupedArgs a{indices, b_values, b_scales, a_values_table, a_scales_table, alpha_table, 1.0f, d, nullptr, table_len, plan->groups,
                  plan->m, plan->k};
    return launch_grouped<kSharedNvfp4, true>(a, stream);
}

cudaError_t infer_cutlass_fp4_grouped_gemv_f32_indexed_a_on_stream(void* raw, const uint32_t* indices,
                                                                   const uint8_t* const* a_values_table,
                                                                   const uint8_t* const* a_scales_table, uint32_t table_len,
                                                                   const uint8_t* b_values, const uint8_t* b_scales, float* const* d,
                                                                   float alpha, cudaStream_t stream) {
    auto* plan = static_cast<GroupedGemvPlan*>(raw);
    if (!plan || !indices || !a_values_table || !a_scales_table || !b_values || !b_scales || !d) return cudaErrorInvalidValue;
    GroupedArgs a{indices, b_values, b_scales, a_values_table, a_scales_table, nullptr, alpha, d, nullptr, table_len, plan->groups, plan->m,
                  plan->k};
    return launch_grouped<kSharedNvfp4, true>(a, stream);
}

cudaError_t infer_cutlass_fp4_grouped_gemv_f32_contiguous_b_on_stream(void* raw, const uint8_t* const* a_values_table,
                                                                      const uint8_t* const* a_scales_table, const uint8_t* b_values,
                                                                      const uint8_t* b_scales, float* d, float alpha,
                                                                      cudaStream_t stream) {
    auto* plan = static_cast<GroupedGemvPlan*>(raw);
    if (!plan || !a_values_table || !a_scales_table || !b_values || !b_scales || !d) return cudaErrorInvalidValue;
    // group g multiplies table entry g with the shared activation row and writes d[g * m ...]
    GroupedArgs a{nullptr, b_values, b_scales, a_values_table, a_scales_table, nullptr, alpha, nullptr, d, plan->groups, plan->groups,
                  plan->m, plan->k};
    return launch_grouped<kSharedNvfp4, true>(a, stream);
}

cudaError_t infer_moe_silu_slots_f32_on_stream(const uint32_t* indices, const float* const* gate_up_table, float* const* output_table,
                                               const float* gate_up_alpha_table, uint32_t rows, uint32_t groups, cudaStream_t stream) {
    if (!indices || !gate_up_table || !output_table || !gate_up_alpha_table || rows == 0 || groups == 0) return cudaErrorInvalidValue;
    silu_slots_f32_kernel<<<dim3((rows + 255) / 256, groups), 256, 0, stream>>>(indices, gate_up_table, output_table, gate_up_alpha_table,
                                                                                rows);
    return cudaGetLastError();
}

cudaError_t infer_moe_silu_quantize_slots_nvfp4_simple_scales_on_stream(const uint32_t* indices, const float* const* gate_up_table,
                                                                        uint8_t* const* packed_table, uint8_t* const* scales_table,
                                                                        const float* input_scale_table,
                                                                        const float* gate_up_alpha_table, uint32_t rows,
                                                                        uint32_t groups, cudaStream_t stream) {
    if (!indices || !gate_up_table || !packed_table || !scales_table || !input_scale_table || !gate_up_alpha_table || rows == 0 ||
        groups == 0)
        return cudaErrorInvalidValue;
    const uint32_t blocks = (rows + 15) / 16;
    silu_quantize_slots_kernel<<<dim3((blocks + 127) / 128, groups), 128, 0, stream>>>(indices, gate_up_table, packed_table, scales_table,
                                                                                      input_scale_table, gate_up_alpha_table, rows);
    return cudaGetLastError();
}

cudaError_t infer_moe_weighted_accumulate_slots_f32_batch_on_stream(const uint32_t* indices, const float* route_weights,
                                                                    const float* const* inputs, const float* alpha_table,
                                                                    float* output, uint32_t rows, uint32_t len, uint32_t groups,
                                                                    cudaStream_t stream) {
    if (!indices || !route_weights || !inputs || !alpha_table || !output || rows == 0 || len == 0 || groups == 0)
        return cudaErrorInvalidValue;
    const size_t total = static_cast<size_t>(rows) * len;
    accumulate_slots_kernel<false><<<static_cast<uint32_t>((total + 255) / 256), 256, 0, stream>>>(
        indices, route_weights, inputs, alpha_table, nullptr, nullptr, nullptr, output, rows, len, groups);
    return cudaGetLastError();
}

cudaError_t infer_moe_weighted_accumulate_slots_f32_on_stream(const uint32_t* indices, const float* route_weights,
                                                              const float* const* inputs, const float* alpha_table, float* output,
                                                              uint32_t len, uint32_t groups, cudaStream_t stream) {
    return infer_moe_weighted_accumulate_slots_f32_batch_on_stream(indices, route_weights, inputs, alpha_table, output, 1, len, groups,
                                                                   stream);
}

cudaError_t infer_qwen36_ffn_finalize_routed_batch_f32_on_stream(const uint32_t* indices, const float* route_weights,
                                                                 const float* const* routed_outputs, const float* alpha_table,
                                                                 const float* shared_gate_logit, const float* shared_output,
                                                                 const float* residual, float* output, uint32_t rows, uint32_t cols,
                                                                 uint32_t groups_per_row, cudaStream_t stream) {
    if (!indices || !route_weights || !routed_outputs || !alpha_table || !shared_gate_logit || !shared_output || !residual || !output ||
        rows == 0 || cols == 0 || groups_per_row == 0)
        return cudaErrorInvalidValue;
    const size_t total = static_cast<size_t>(rows) * cols;
    accumulate_slots_kernel<true><<<static_cast<uint32_t>((total + 255) / 256), 256, 0, stream>>>(
        indices, route_weights, routed_outputs, alpha_table, shared_gate_logit, shared_output, residual, output, rows, cols, groups_per_row);
    return cudaGetLastError();
}

cudaError_t infer_qwen36_ffn_finalize_routed_f32_on_stream(const uint32_t* indices, const float* route_weights,
                                                           const float* const* routed_outputs, const float* alpha_table,
                                                           const float* shared_gate_logit, const float* shared_output,
                                                           const float* residual, float* output, uint32_t len, uint32_t groups,
                                                           cudaStream_t stream) {
    return infer_qwen36_ffn_finalize_routed_batch_f32_on_stream(indices, route_weights, routed_outputs, alpha_table, shared_gate_logit,
                                                                shared_output, residual, output, 1, len, groups, stream);
}

/* crates/eider-cuda/src/ffi.rs:3473 (kernels non_gemm.cu:13423-13482, 8287-8328): arg-max over the lm-head logits without
 * writing them.  scratch_value / scratch_index hold scratch_len per-CTA candidates; any scratch_len >= 1 works here (the
 * CTAs walk the rows), up to 1024 entries are used.  warps_per_block is the reference's launch width and must be one of
 * its values (4, 8, 16, 32); this implementation needs in_features % 32 == 0. */
cudaError_t infer_nvfp4_w4a16_top1_f32_on_stream(const float* input, const uint8_t* packed_weight, const uint8_t* weight_scale,
                                                 float* scratch_value, uint32_t* scratch_index, uint32_t scratch_len,
                                                 uint32_t* out_index, float* out_value, uint32_t out_features, uint32_t in_features,
                                                 float weight_scale_2, uint32_t warps_per_block, cudaStream_t stream) {
    if (!input || !packed_weight || !weight_scale || !scratch_value || !scratch_index || !out_index || !out_value ||
        out_features == 0 || in_features == 0 || in_features % 32 != 0 || !isfinite(weight_scale_2) || scratch_len == 0 ||
        (warps_per_block != 4 && warps_per_block != 8 && warps_per_block != 16 && warps_per_block != 32))
        return cudaErrorInvalidValue;
    const size_t smem = static_cast<size_t>(in_features) * sizeof(float);
    if (smem > 200 * 1024) return cudaErrorNotSupported;
    if (smem > 48 * 1024) {
        cudaError_t st = cudaFuncSetAttribute(top1_pass1_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        if (st != cudaSuccess) return st;
    }
    uint32_t blocks = (out_features + kWarps - 1) / kWarps;
    if (blocks > 1024) blocks = 1024;
    if (blocks > scratch_len) blocks = scratch_len;
    top1_pass1_kernel<<<blocks, kWarps * 32, smem, stream>>>(input, packed_weight, weight_scale, weight_scale_2, out_features, in_features,
                                                             scratch_value, scratch_index);
    cudaError_t st = cudaGetLastError();
    if (st != cudaSuccess) return st;
    top1_pass2_kernel<<<1, 256, 0, stream>>>(scratch_value, scratch_index, blocks, out_index, out_value);
    return cudaGetLastError();
}

}  // extern "C"
