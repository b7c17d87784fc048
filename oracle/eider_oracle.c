/*
 * CPU oracle for Eider's quantized-linear path.  TEST INFRASTRUCTURE ONLY:
 * nothing in the shipped library links or calls this file; it exists so the
 * CUDA kernels can be checked against a plain restatement of the reference's
 * host-side numerics.
 *
 * Parity status: PINNED.  The codecs are checked against the reference's own
 * known-answer vectors (crates/eider-cuda/src/format.rs:395-527,
 * crates/eider-format/src/modelopt.rs:1281-1330) and against the reference's
 * C++ conversion oracle (crates/eider-cuda/native/fp4_oracle.cpp) compiled
 * from where it lies into oracle/_ref/ by oracle/Makefile.
 *
 * Every function cites the reference file:line it restates.  Plain C99 with
 * pthreads on the outer loops of the bulk routines (results do not depend on
 * the thread count: each output element is reduced by one thread in K order).
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include <pthread.h>
#include <unistd.h>

#define ORACLE_API __attribute__((visibility("default")))


/* ------------------------------------------------------------ thread helper */

static int g_threads = 0; /* 0 = all online cores */

ORACLE_API void oracle_set_threads(int threads) { g_threads = threads; }

ORACLE_API int oracle_max_threads(void) {
    if (g_threads > 0) return g_threads;
    long n = sysconf(_SC_NPROCESSORS_ONLN);
    return n > 0 ? (int)n : 1;
}

typedef void (*range_fn)(size_t begin, size_t end, void* ctx);
typedef struct { range_fn fn; void* ctx; size_t begin, end; } range_job;

static void* range_trampoline(void* arg) {
    range_job* j = (range_job*)arg;
    j->fn(j->begin, j->end, j->ctx);
    return NULL;
}

/* Static split of [0, n) over the configured thread count. */
static void parallel_for(size_t n, range_fn fn, void* ctx) {
    int threads = oracle_max_threads();
    if ((size_t)threads > n) threads = (int)(n ? n : 1);
    if (threads <= 1) { fn(0, n, ctx); return; }
    pthread_t* tid = (pthread_t*)malloc(sizeof(pthread_t) * (size_t)threads);
    char* live = (char*)calloc((size_t)threads, 1);
    range_job* jobs = (range_job*)malloc(sizeof(range_job) * (size_t)threads);
    size_t chunk = (n + (size_t)threads - 1) / (size_t)threads;
    for (int t = 0; t < threads; ++t) {
        size_t b = (size_t)t * chunk, e = b + chunk < n ? b + chunk : n;
        if (b >= e) break;
        jobs[t].fn = fn; jobs[t].ctx = ctx; jobs[t].begin = b; jobs[t].end = e;
        if (pthread_create(&tid[t], NULL, range_trampoline, &jobs[t]) == 0) live[t] = 1;
        else fn(b, e, ctx);
    }
    for (int t = 0; t < threads; ++t) if (live[t]) pthread_join(tid[t], NULL);
    free(tid);
    free(live);
    free(jobs);
}

/* ------------------------------------------------------------------ codecs */

static const float kE2M1[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};

/* crates/eider-cuda/src/format.rs:44-75 (duplicate: crates/eider-format/src/modelopt.rs:1163-1190).
 * NaN -> 0x7; sign kept on -0; |v|>6 saturates; nearest with ties to the even code. */
ORACLE_API uint8_t oracle_e2m1_code(float value) {
    if (isnan(value)) return 0x7;
    uint8_t sign = signbit(value) ? 0x8 : 0x0;
    float a = fabsf(value);
    if (a > 6.0f) return sign | 0x7;
    uint8_t best = 0;
    float best_err = INFINITY;
    for (uint8_t code = 0; code < 8; ++code) {
        float err = fabsf(a - kE2M1[code]);
        if (err < best_err || (err == best_err && (code & 1) == 0 && (best & 1) == 1)) {
            best = code;
            best_err = err;
        }
    }
    return sign | best;
}

/* crates/eider-cuda/src/format.rs:78-96 */
ORACLE_API float oracle_e2m1_value(uint8_t code) {
    float m = kE2M1[code & 7];
    return (code & 8) ? -m : m;
}

/* crates/eider-cuda/src/format.rs:121-133 */
ORACLE_API float oracle_e4m3_value(uint8_t code) {
    float sign = (code & 0x80) ? -1.0f : 1.0f;
    int exp = (code >> 3) & 0x0f;
    int mant = code & 7;
    if (exp == 0) return sign * (float)mant * ldexpf(1.0f, -9);
    if (exp == 0x0f && mant == 7) return NAN;
    return sign * (1.0f + (float)mant / 8.0f) * ldexpf(1.0f, exp - 7);
}

/* crates/eider-cuda/src/format.rs:139-145 */
ORACLE_API float oracle_e8m0_value(uint8_t code) {
    if (code == 0xff) return NAN;
    return ldexpf(1.0f, (int)code - 127);
}

/* crates/eider-cuda/src/format.rs:151-167: exhaustive nearest search over
 * 0x01..0x7e starting from code 0, ties to the even code, saturates at 448. */
ORACLE_API uint8_t oracle_ue4m3_code(float value) {
    if (!isfinite(value) || value <= 0.0f) return 0;
    uint8_t best = 0;
    float best_err = fabsf(value);
    for (int code = 1; code <= 0x7e; ++code) {
        float err = fabsf(value - oracle_e4m3_value((uint8_t)code));
        if (err < best_err || (err == best_err && (code & 1) == 0 && (best & 1) == 1)) {
            best = (uint8_t)code;
            best_err = err;
        }
    }
    return best;
}

/* crates/eider-cuda/src/format.rs:173-183 */
ORACLE_API uint8_t oracle_e4m3_code(float value) {
    if (!isfinite(value) || value == 0.0f) return 0;
    uint8_t mag = oracle_ue4m3_code(fabsf(value));
    return signbit(value) ? (mag | 0x80) : mag;
}

/* crates/eider-cuda/src/format.rs:362-376 */
ORACLE_API float oracle_bf16_to_f32(uint16_t bits) {
    uint32_t u = (uint32_t)bits << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

ORACLE_API uint16_t oracle_f32_to_bf16(float value) {
    uint32_t bits;
    memcpy(&bits, &value, 4);
    uint32_t lsb = (bits >> 16) & 1u;
    uint32_t rounded = bits + 0x7fffu + lsb;
    return (uint16_t)(rounded >> 16);
}

/* crates/eider-cuda/src/format.rs:101-110: element 2i in the low nibble. */
ORACLE_API void oracle_pack_e2m1(const float* values, size_t n, uint8_t* packed) {
    for (size_t i = 0; i < n; i += 2) {
        uint8_t lo = oracle_e2m1_code(values[i]);
        uint8_t hi = (i + 1 < n) ? oracle_e2m1_code(values[i + 1]) : 0;
        packed[i / 2] = (uint8_t)(lo | (hi << 4));
    }
}

/* ------------------------------------------------------- tiled scale layout */

/* crates/eider-cuda/src/format.rs:194-198 */
ORACLE_API size_t oracle_scale_layout_len(size_t outer_dim, size_t inner_dim) {
    size_t blocks = (inner_dim + 15) / 16;
    size_t padded = (blocks + 3) / 4 * 4;
    return (outer_dim + 127) / 128 * 128 * padded;
}

/* crates/eider-cuda/src/format.rs:208-218 */
ORACLE_API size_t oracle_tiled_scale_offset(size_t outer, size_t inner_block, size_t inner_dim) {
    size_t blocks = (inner_dim + 15) / 16;
    size_t padded = (blocks + 3) / 4 * 4;
    size_t tile_outer = outer / 128, in_tile = outer % 128;
    size_t tile_inner = inner_block / 4, in_inner = inner_block % 4;
    size_t base = (tile_inner * 4 + tile_outer * padded) * 128;
    return base + (in_tile % 32) * 16 + (in_tile / 32) * 4 + in_inner;
}

/* crates/eider-format/src/modelopt.rs:1148-1161: row-major [N][K/16] -> tiled. */
ORACLE_API void oracle_scales_to_tiled(const uint8_t* row_major, size_t out_features,
                                       size_t in_features, uint8_t* tiled) {
    size_t blocks = in_features / 16;
    memset(tiled, 0, oracle_scale_layout_len(out_features, in_features));
    for (size_t o = 0; o < out_features; ++o)
        for (size_t b = 0; b < blocks; ++b)
            tiled[oracle_tiled_scale_offset(o, b, in_features)] = row_major[o * blocks + b];
}

/* --------------------------------------------------- NVFP4 activation quantize */

/* One token row.  Device order of operations, crates/eider-cuda/native/non_gemm.cu:106-155
 * (== host crates/eider-cuda/src/format.rs:242-292 when input_scale == 1):
 *   v = x / input_scale; amax over finite v; sc = ue4m3(amax / 6); code = e2m1(v / e4m3(sc)).
 * `scale_out[b]` receives block b's scale byte; packed gets K/2 bytes (odd tail: high nibble 0). */
static void quantize_row(const float* x, size_t k, float input_scale, uint8_t* packed,
                         uint8_t* scale_out) {
    size_t blocks = (k + 15) / 16;
    for (size_t b = 0; b < blocks; ++b) {
        size_t start = b * 16, end = start + 16 < k ? start + 16 : k;
        float amax = 0.0f;
        for (size_t i = start; i < end; ++i) {
            float v = x[i] / input_scale;
            if (isfinite(v)) amax = fmaxf(amax, fabsf(v));
        }
        uint8_t sc = amax == 0.0f ? 0 : oracle_ue4m3_code(amax / 6.0f);
        float s = oracle_e4m3_value(sc);
        scale_out[b] = sc;
        for (size_t i = start; i < end; ++i) {
            float v = s == 0.0f ? 0.0f : (x[i] / input_scale) / s;
            uint8_t code = oracle_e2m1_code(v);
            if ((i & 1) == 0) packed[i / 2] = code;
            else packed[i / 2] |= (uint8_t)(code << 4);
        }
    }
}

/* Activation quantize, scalar static input scale: the reference operator
 * infer_quantize_nvfp4_col_major_f32 (non_gemm.cu:106-191).  x is [tokens][k] f32
 * ("col-major K x tokens"), scales land in the tiled layout with outer = token.
 * `scales` must hold oracle_scale_layout_len(tokens, k) bytes; padding is zeroed. */
ORACLE_API void oracle_quantize_nvfp4(const float* x, size_t tokens, size_t k, float input_scale,
                                      uint8_t* packed, uint8_t* scales) {
    size_t blocks = (k + 15) / 16;
    memset(scales, 0, oracle_scale_layout_len(tokens, k));
    uint8_t* tmp = (uint8_t*)malloc(blocks);
    for (size_t t = 0; t < tokens; ++t) {
        quantize_row(x + t * k, k, input_scale, packed + t * (k / 2), tmp);
        for (size_t b = 0; b < blocks; ++b) scales[oracle_tiled_scale_offset(t, b, k)] = tmp[b];
    }
    free(tmp);
}

/* Row scale of the on-the-fly quantizer: the smallest power of two g with amax / g <= 2688 (= 6 * 448, so the
 * largest block scale still fits E4M3), 1 for amax == 0, clamped to the normal range.  A power of two makes
 * x / g exact.  2688 = 1.3125 * 2^11, so g = 2^(e - 11) when the significand of amax is <= 1.3125, else 2^(e - 10). */
ORACLE_API float oracle_row_scale(float amax) {
    if (!(amax > 0.0f)) return 1.0f;
    uint32_t bits;
    memcpy(&bits, &amax, 4);
    int e = (int)(bits >> 23);
    uint32_t mant = bits & 0x7fffffu;
    int ge = e - 11 + (mant > 0x280000u ? 1 : 0);
    if (ge < 1) ge = 1;
    if (ge > 254) ge = 254;
    uint32_t gb = (uint32_t)ge << 23;
    float g;
    memcpy(&g, &gb, 4);
    return g;
}

/* Per-row global scale (the on-the-fly quantizer of the prefill GEMM configs; not a
 * reference operator): g_t = oracle_row_scale(amax_t) over the finite entries of the row,
 * then the reference quantizer above with input_scale = g_t. */
ORACLE_API void oracle_quantize_nvfp4_rowscale(const float* x, size_t tokens, size_t k,
                                               uint8_t* packed, uint8_t* scales,
                                               float* row_scales) {
    size_t blocks = (k + 15) / 16;
    memset(scales, 0, oracle_scale_layout_len(tokens, k));
    uint8_t* tmp = (uint8_t*)malloc(blocks);
    for (size_t t = 0; t < tokens; ++t) {
        float amax = 0.0f;
        for (size_t i = 0; i < k; ++i) {
            float v = x[t * k + i];
            if (isfinite(v)) amax = fmaxf(amax, fabsf(v));
        }
        float g = oracle_row_scale(amax);
        row_scales[t] = g;
        quantize_row(x + t * k, k, g, packed + t * (k / 2), tmp);
        for (size_t b = 0; b < blocks; ++b) scales[oracle_tiled_scale_offset(t, b, k)] = tmp[b];
    }
    free(tmp);
}

/* ModelOpt weight record from f32 values, row-major [N][K]:
 * crates/eider-format/src/modelopt.rs:649-716 is the g == 1 case; a checkpoint made by
 * ModelOpt carries weight_scale_2 = g = amax(W)/(6*448) and block scales relative to it
 * (modelopt.rs:143-170 consumes that form).  Same arithmetic as the activation path with
 * input_scale = g; scales stay row-major [N][K/16]. */
typedef struct { const float* w; size_t k; float g; uint8_t* packed; uint8_t* scales; } qw_ctx;
static void qw_body(size_t b, size_t e, void* p) {
    qw_ctx* c = (qw_ctx*)p;
    size_t blocks = c->k / 16;
    for (size_t r = b; r < e; ++r)
        quantize_row(c->w + r * c->k, c->k, c->g, c->packed + r * (c->k / 2), c->scales + r * blocks);
}
ORACLE_API void oracle_quantize_weight(const float* w, size_t n, size_t k, float global_scale,
                                       uint8_t* packed, uint8_t* scales_row_major) {
    qw_ctx c = {w, k, global_scale, packed, scales_row_major};
    parallel_for(n, qw_body, &c);
}

/* g = amax(W) / (6 * 448), single IEEE divide by 2688. */
ORACLE_API float oracle_weight_global_scale(const float* w, size_t count) {
    float amax = 0.0f;
    for (size_t i = 0; i < count; ++i)
        if (isfinite(w[i])) amax = fmaxf(amax, fabsf(w[i]));
    return amax == 0.0f ? 1.0f : amax / 2688.0f;
}

/* ----------------------------------------------------------------- dequantize */

typedef struct { const uint8_t* packed; const uint8_t* scales; size_t k; float* out; int tiled; float mul; } dq_ctx;
static void dq_body(size_t b, size_t e, void* p) {
    dq_ctx* c = (dq_ctx*)p;
    size_t k = c->k, blocks = k / 16;
    for (size_t r = b; r < e; ++r)
        for (size_t i = 0; i < k; ++i) {
            size_t flat = r * k + i;
            uint8_t nib = (flat & 1) ? (c->packed[flat / 2] >> 4) : (c->packed[flat / 2] & 0x0f);
            uint8_t sc = c->tiled ? c->scales[oracle_tiled_scale_offset(r, i / 16, k)]
                                  : c->scales[r * blocks + i / 16];
            float v = oracle_e2m1_value(nib) * oracle_e4m3_value(sc);
            c->out[flat] = c->mul == 1.0f ? v : v * c->mul;
        }
}

/* crates/eider-format/src/modelopt.rs:741-757: e2m1(code) * e4m3(scale[n][k/16]); the
 * per-tensor weight_scale_2 is NOT applied here (the caller folds it into alpha).
 * Output row-major [N][K] (the reference calls the same memory "col-major K x N"). */
ORACLE_API void oracle_dequantize_rowmajor_scales(const uint8_t* packed, const uint8_t* scales,
                                                  size_t n, size_t k, float* out) {
    dq_ctx c = {packed, scales, k, out, 0, 1.0f};
    parallel_for(n, dq_body, &c);
}

/* Same for tiled scales (activations): crates/eider-cuda/src/format.rs:283-285. */
ORACLE_API void oracle_dequantize_tiled_scales(const uint8_t* packed, const uint8_t* scales,
                                               size_t outer, size_t k, float* out) {
    dq_ctx c = {packed, scales, k, out, 1, 1.0f};
    parallel_for(outer, dq_body, &c);
}

/* --------------------------------------------------------------------- matmul */

typedef struct { const float* a; const float* w; size_t m, n, k; float alpha;
                 const float* row_scale; const float* col_scale; float* y; } mm_ctx;
static void mm_body(size_t b, size_t e, void* p) {
    mm_ctx* c = (mm_ctx*)p;
    for (size_t col = b; col < e; ++col)
        for (size_t row = 0; row < c->m; ++row) {
            float acc = 0.0f;
            const float* ar = c->a + row * c->k;
            const float* wr = c->w + col * c->k;
            for (size_t i = 0; i < c->k; ++i) acc += ar[i] * wr[i];
            float s = c->alpha;
            if (c->row_scale) s *= c->row_scale[row];
            if (c->col_scale) s *= c->col_scale[col];
            c->y[row * c->n + col] = acc * s;
        }
}

/* y[t][n] = alpha * row_scale[t] * col_scale[n] * sum_k a[t][k] * w[n][k], fp32 accumulate in
 * K order (crates/eider-cuda/src/format.rs:379-392 restated for the K-contiguous images;
 * alpha as in crates/eider-cuda/src/cublaslt/fp4_tn.rs:1527-1528).  row_scale / col_scale may
 * be NULL (== 1). */
ORACLE_API void oracle_matmul_nt(const float* a, const float* w, size_t m, size_t n, size_t k,
                                 float alpha, const float* row_scale, const float* col_scale,
                                 float* y) {
    mm_ctx c = {a, w, m, n, k, alpha, row_scale, col_scale, y};
    parallel_for(n, mm_body, &c);
}

/* The reference's host path for an NVFP4 linear, literally: unpack the record to f32
 * (modelopt.rs:741-757), multiply by weight_scale_2, then the f32 triple loop
 * (format.rs:379-392).  Used as the timed CPU baseline.  `threads` <= 0 keeps the configured
 * count (all cores); 1 gives the reference's single-threaded form.  `scratch` holds n*k floats. */
ORACLE_API void oracle_nvfp4_linear_host(const float* x, size_t m, const uint8_t* packed,
                                         const uint8_t* scales_row_major, float weight_scale_2,
                                         size_t n, size_t k, float* scratch, float* y,
                                         int threads) {
    int saved = g_threads;
    if (threads > 0) g_threads = threads;
    dq_ctx c = {packed, scales_row_major, k, scratch, 0, weight_scale_2};
    parallel_for(n, dq_body, &c);
    oracle_matmul_nt(x, scratch, m, n, k, 1.0f, NULL, NULL, y);
    g_threads = saved;
}

/* ------------------------------------------------------------------------ FP8 */

/* __nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3) as the reference's device quantizers call
 * it (crates/eider-cuda/native/non_gemm.cu:9971-9972): NaN -> 0x7f, |v| > 448 (and +-inf)
 * saturate to +-448, -0 keeps its sign, finite values round to nearest even. */
ORACLE_API uint8_t oracle_e4m3_satfinite(float v) {
    if (isnan(v)) return 0x7f;
    uint8_t sign = signbit(v) ? 0x80 : 0;
    float a = fabsf(v);
    if (isinf(a)) return sign | 0x7e;
    return sign | oracle_ue4m3_code(a);
}

/* Per-token dynamic E4M3 quantize: crates/eider-cuda/native/non_gemm.cu:9952-9974,
 * 10028-10066.  s = amax/448 over the finite entries (1 when amax == 0);
 * q = cvt_satfinite(x / s). */
ORACLE_API void oracle_quantize_fp8_dynamic(const float* x, size_t rows, size_t cols, uint8_t* q,
                                            float* row_scale) {
    for (size_t r = 0; r < rows; ++r) {
        float amax = 0.0f;
        for (size_t i = 0; i < cols; ++i)
            if (isfinite(x[r * cols + i])) amax = fmaxf(amax, fabsf(x[r * cols + i]));
        float s = amax == 0.0f ? 1.0f : amax / 448.0f;
        row_scale[r] = s;
        for (size_t i = 0; i < cols; ++i) q[r * cols + i] = oracle_e4m3_satfinite(x[r * cols + i] / s);
    }
}

/* Static-scale form: crates/eider-cuda/native/non_gemm.cu:10487+ (q = cvt_satfinite(x / input_scale)). */
ORACLE_API void oracle_quantize_fp8_static(const float* x, size_t len, float input_scale,
                                           uint8_t* q) {
    for (size_t i = 0; i < len; ++i) q[i] = oracle_e4m3_satfinite(x[i] / input_scale);
}

typedef struct { const float* w; size_t k; uint8_t* q; float* cs; } f8w_ctx;
static void f8w_body(size_t b, size_t e, void* p) {
    f8w_ctx* c = (f8w_ctx*)p;
    size_t k = c->k;
    for (size_t r = b; r < e; ++r) {
        float amax = 0.0f;
        for (size_t i = 0; i < k; ++i)
            if (isfinite(c->w[r * k + i])) amax = fmaxf(amax, fabsf(c->w[r * k + i]));
        float s = amax == 0.0f ? 1.0f : amax / 448.0f;
        c->cs[r] = s;
        for (size_t i = 0; i < k; ++i) c->q[r * k + i] = oracle_e4m3_satfinite(c->w[r * k + i] / s);
    }
}

/* Per-output-channel weight quantize: s_w[n] = amax_n / 448 (1 when 0);
 * code = e4m3(w / s_w) (precedent crates/infer/src/qwen3/qwen36.rs:2047-2057). */
ORACLE_API void oracle_quantize_fp8_weight(const float* w, size_t n, size_t k, uint8_t* q,
                                           float* channel_scale) {
    f8w_ctx c = {w, k, q, channel_scale};
    parallel_for(n, f8w_body, &c);
}

typedef struct { const uint8_t* xq; const float* s_x; const uint8_t* wq; const float* s_w;
                 size_t m, n, k; float* y; const float* lut; } f8l_ctx;
static void f8l_body(size_t b, size_t e, void* p) {
    f8l_ctx* c = (f8l_ctx*)p;
    for (size_t col = b; col < e; ++col)
        for (size_t row = 0; row < c->m; ++row) {
            float acc = 0.0f;
            for (size_t i = 0; i < c->k; ++i)
                acc += c->lut[c->xq[row * c->k + i]] * c->lut[c->wq[col * c->k + i]];
            c->y[row * c->n + col] = acc * c->s_x[row] * c->s_w[col];
        }
}

/* y[t][n] = (sum_k e4m3(xq[t][k]) * e4m3(w[n][k])) * s_x[t] * s_w[n]
 * (crates/eider-cuda/native/non_gemm.cu:9976-10011; host twin
 * crates/eider-cuda/src/kernels/non_gemm.rs:25067-25083). */
ORACLE_API void oracle_fp8_linear(const uint8_t* xq, const float* s_x, const uint8_t* wq,
                                  const float* s_w, size_t m, size_t n, size_t k, float* y) {
    float lut[256];
    for (int i = 0; i < 256; ++i) lut[i] = oracle_e4m3_value((uint8_t)i);
    f8l_ctx c = {xq, s_x, wq, s_w, m, n, k, y, lut};
    parallel_for(n, f8l_body, &c);
}

/* ------------------------------------------------------------------------ MoE */

static float sanitize_logit(float v) {
    if (isnan(v)) return -INFINITY;
    if (v == INFINITY) return 3.402823466e+38f;
    return v;
}

/* Router top-k: crates/eider-cuda/native/non_gemm.cu:1854-2020.  Strict '>' insertion, so
 * equal values keep ascending expert order; renormalised mode = softmax over the selected
 * logits; otherwise full softmax, then top-k of the probabilities. */
ORACLE_API void oracle_moe_topk(const float* logits, size_t tokens, size_t experts, size_t k,
                                int norm_topk_prob, uint32_t* out_idx, float* out_w) {
    float* probs = (float*)malloc(experts * sizeof(float));
    for (size_t t = 0; t < tokens; ++t) {
        const float* lg = logits + t * experts;
        uint32_t* idx = out_idx + t * k;
        float* w = out_w + t * k;
        if (!norm_topk_prob) {
            float mx = -INFINITY;
            for (size_t e = 0; e < experts; ++e) mx = fmaxf(mx, sanitize_logit(lg[e]));
            if (!isfinite(mx)) {
                for (size_t s = 0; s < k; ++s) { idx[s] = (uint32_t)s; w[s] = s == 0 ? 1.0f : 0.0f; }
                continue;
            }
            float sum = 0.0f;
            for (size_t e = 0; e < experts; ++e) {
                probs[e] = expf(sanitize_logit(lg[e]) - mx);
                sum += probs[e];
            }
            for (size_t e = 0; e < experts; ++e) probs[e] = probs[e] / sum;
        }
        for (size_t s = 0; s < k; ++s) { idx[s] = 0xffffffffu; w[s] = -INFINITY; }
        for (size_t e = 0; e < experts; ++e) {
            float v = norm_topk_prob ? sanitize_logit(lg[e]) : probs[e];
            for (size_t s = 0; s < k; ++s) {
                if (v > w[s]) {
                    for (size_t mv = k - 1; mv > s; --mv) { idx[mv] = idx[mv - 1]; w[mv] = w[mv - 1]; }
                    idx[s] = (uint32_t)e;
                    w[s] = v;
                    break;
                }
            }
        }
        if (norm_topk_prob) {
            if (!isfinite(w[0])) {
                for (size_t s = 0; s < k; ++s) { idx[s] = (uint32_t)s; w[s] = s == 0 ? 1.0f : 0.0f; }
                continue;
            }
            float mx = w[0], sum = 0.0f;
            for (size_t s = 0; s < k; ++s) { w[s] = expf(w[s] - mx); sum += w[s]; }
            if (sum > 0.0f && isfinite(sum))
                for (size_t s = 0; s < k; ++s) w[s] /= sum;
        }
    }
    free(probs);
}

/* Permute metadata: crates/eider-cuda/native/non_gemm.cu:2473-2550.  The reference scatters
 * with atomics (order inside an expert unspecified); this restatement uses ascending route
 * order inside each expert, which is one of the orders the reference may produce. */
ORACLE_API void oracle_moe_sort_routes(const uint32_t* indices, size_t routes, size_t experts,
                                       uint32_t* counts, uint32_t* offsets, uint32_t* sorted_routes,
                                       uint32_t* sorted_experts, uint32_t* route_to_sorted) {
    memset(counts, 0, experts * sizeof(uint32_t));
    for (size_t r = 0; r < routes; ++r)
        if (indices[r] < experts) counts[indices[r]]++;
    uint32_t off = 0;
    uint32_t* cursor = (uint32_t*)malloc(experts * sizeof(uint32_t));
    for (size_t e = 0; e < experts; ++e) { offsets[e] = off; cursor[e] = off; off += counts[e]; }
    offsets[experts] = off;
    for (size_t r = 0; r < routes; ++r) {
        uint32_t e = indices[r];
        if (e >= experts) continue;
        uint32_t s = cursor[e]++;
        sorted_routes[s] = (uint32_t)r;
        sorted_experts[s] = e;
        route_to_sorted[r] = s;
    }
    free(cursor);
}

/* non_gemm.cu:2554-2557 */
ORACLE_API size_t oracle_moe_scale_base(uint32_t expert, const uint32_t* offsets,
                                        size_t scale_tile_bytes) {
    return (((size_t)offsets[expert] + 127) / 128 + expert) * scale_tile_bytes;
}

/* Gather token rows into expert-major order and quantize with unit global scale:
 * crates/eider-cuda/native/non_gemm.cu:2621-2703.  packed is [routes][K/2]; each expert's
 * scales start at oracle_moe_scale_base and are tiled with outer = row inside the expert.
 * `scales` must be zeroed by the caller over its whole length. */
ORACLE_API void oracle_moe_gather_quantize(const float* x, const uint32_t* sorted_routes,
                                           const uint32_t* sorted_experts, const uint32_t* offsets,
                                           size_t routes, size_t routes_per_row, size_t k,
                                           size_t scale_tile_bytes, int gather_rows,
                                           uint8_t* packed, uint8_t* scales) {
    size_t blocks = (k + 15) / 16;
    uint8_t* tmp = (uint8_t*)malloc(blocks);
    for (size_t s = 0; s < routes; ++s) {
        size_t src = gather_rows ? sorted_routes[s] / routes_per_row : s;
        uint32_t e = sorted_experts[s];
        size_t col = s - offsets[e];
        quantize_row(x + src * k, k, 1.0f, packed + s * (k / 2), tmp);
        size_t base = oracle_moe_scale_base(e, offsets, scale_tile_bytes);
        for (size_t b = 0; b < blocks; ++b) scales[base + oracle_tiled_scale_offset(col, b, k)] = tmp[b];
    }
    free(tmp);
}

/* silu(gate) * up on bf16 halves, then the same quantizer:
 * crates/eider-cuda/native/non_gemm.cu:2805-2875 (gate = first half of the row, up = second;
 * silu = g / (1 + expf(-g)); product in fp32).  `act_out` (may be NULL) receives the fp32
 * products so a caller can compare kernels that use a different expf. */
ORACLE_API void oracle_moe_silu_mul_quantize(const uint16_t* gate_up, const uint32_t* sorted_experts,
                                             const uint32_t* offsets, size_t routes, size_t k,
                                             size_t scale_tile_bytes, uint8_t* packed,
                                             uint8_t* scales, float* act_out) {
    size_t blocks = k / 16;
    uint8_t* tmp = (uint8_t*)malloc(blocks);
    float* row = (float*)malloc(k * sizeof(float));
    for (size_t s = 0; s < routes; ++s) {
        const uint16_t* g = gate_up + s * k * 2;
        const uint16_t* u = g + k;
        for (size_t i = 0; i < k; ++i) {
            float gv = oracle_bf16_to_f32(g[i]);
            float silu = gv / (1.0f + expf(-gv));
            row[i] = silu * oracle_bf16_to_f32(u[i]);
        }
        if (act_out) memcpy(act_out + s * k, row, k * sizeof(float));
        uint32_t e = sorted_experts[s];
        size_t col = s - offsets[e];
        quantize_row(row, k, 1.0f, packed + s * (k / 2), tmp);
        size_t base = oracle_moe_scale_base(e, offsets, scale_tile_bytes);
        for (size_t b = 0; b < blocks; ++b) scales[base + oracle_tiled_scale_offset(col, b, k)] = tmp[b];
    }
    free(tmp);
    free(row);
}

/* Fused SiLU(gate) * up -> NVFP4 quantize of `tokens` activation rows (the producer in front of the down projection):
 * crates/eider-cuda/native/non_gemm.cu:559-629 (one token: gate = gate_up[0..k), up = gate_up[k..2k),
 * sigmoid = 1 / (1 + expf(-g)), value = g * sigmoid * up, then the activation quantizer with `input_scale`;
 * scales tiled with outer = token).  `act_out` (may be NULL) receives the fp32 products. */
ORACLE_API void oracle_silu_mul_halves_quantize_nvfp4(const float* gate_up, size_t tokens, size_t k, float input_scale,
                                                      uint8_t* packed, uint8_t* scales, float* act_out) {
    size_t blocks = (k + 15) / 16;
    uint8_t* tmp = (uint8_t*)malloc(blocks);
    float* row = (float*)malloc(k * sizeof(float));
    for (size_t t = 0; t < tokens; ++t) {
        const float* g = gate_up + t * 2 * k;
        const float* u = g + k;
        for (size_t i = 0; i < k; ++i) {
            float sigmoid = 1.0f / (1.0f + expf(-g[i]));
            row[i] = g[i] * sigmoid * u[i];
        }
        if (act_out) memcpy(act_out + t * k, row, k * sizeof(float));
        quantize_row(row, k, input_scale, packed + t * ((k + 1) / 2), tmp);
        for (size_t b = 0; b < blocks; ++b) scales[oracle_tiled_scale_offset(t, b, k)] = tmp[b];
    }
    free(tmp);
    free(row);
}

/* Fused RMSNorm -> NVFP4 quantize: crates/eider-cuda/native/non_gemm.cu:193-288
 * (inverse_rms = rsqrtf(sum(x^2) / cols + eps); value = x * inverse_rms * weight / input_scale in that order; block
 * maximum over |value| without a finiteness test; then scale byte and codes as in the activation quantizer).  The
 * reference sums the squares in a thread-strided tree whose order depends on the launch shape; this restatement sums
 * in double and rounds once, so a device result may differ from it by an ulp of inverse_rms.  `norm_out` may be NULL. */
ORACLE_API void oracle_rms_norm_quantize_nvfp4(const float* input, const float* weight, size_t rows, size_t cols, float eps,
                                               float input_scale, uint8_t* packed, uint8_t* scales, float* norm_out) {
    size_t blocks = (cols + 15) / 16;
    float* row = (float*)malloc(cols * sizeof(float));
    for (size_t r = 0; r < rows; ++r) {
        const float* x = input + r * cols;
        double ss = 0.0;
        for (size_t i = 0; i < cols; ++i) ss += (double)x[i] * (double)x[i];
        float mean = (float)ss / (float)cols + eps;
        float inv = 1.0f / sqrtf(mean);
        for (size_t i = 0; i < cols; ++i) row[i] = x[i] * inv * weight[i] / input_scale;
        if (norm_out) memcpy(norm_out + r * cols, row, cols * sizeof(float));
        uint8_t* prow = packed + r * ((cols + 1) / 2);
        for (size_t b = 0; b < blocks; ++b) {
            size_t start = b * 16, end = start + 16 < cols ? start + 16 : cols;
            float amax = 0.0f;
            for (size_t i = start; i < end; ++i) amax = fmaxf(amax, fabsf(row[i]));
            uint8_t sc = amax == 0.0f ? 0 : oracle_ue4m3_code(amax / 6.0f);
            float sv = oracle_e4m3_value(sc);
            scales[oracle_tiled_scale_offset(r, b, cols)] = sc;
            for (size_t i = start; i < end; ++i) {
                uint8_t code = oracle_e2m1_code(sv == 0.0f ? 0.0f : row[i] / sv);
                if ((i & 1) == 0) prow[i / 2] = code;
                else prow[i / 2] |= (uint8_t)(code << 4);
            }
        }
    }
    free(row);
}

/* RMSNorm -> NVFP4 with a second, residual NVFP4 term: crates/eider-cuda/native/non_gemm.cu:290-419.  The primary term
 * is oracle_rms_norm_quantize_nvfp4; residual_i = value_i - e2m1(code_i) * scale (one FMA in the reference's build) is
 * quantized per block with its own scale byte (block maximum over |residual|, no finiteness test). */
ORACLE_API void oracle_rms_norm_quantize_nvfp4_pair(const float* input, const float* weight, size_t rows, size_t cols, float eps,
                                                    float input_scale, uint8_t* packed, uint8_t* scales,
                                                    uint8_t* residual_packed, uint8_t* residual_scales) {
    size_t blocks = (cols + 15) / 16;
    float* norm = (float*)malloc(rows * cols * sizeof(float));
    oracle_rms_norm_quantize_nvfp4(input, weight, rows, cols, eps, input_scale, packed, scales, norm);
    for (size_t r = 0; r < rows; ++r) {
        const uint8_t* prow = packed + r * ((cols + 1) / 2);
        uint8_t* rrow = residual_packed + r * ((cols + 1) / 2);
        for (size_t b = 0; b < blocks; ++b) {
            size_t start = b * 16, end = start + 16 < cols ? start + 16 : cols;
            float sv = oracle_e4m3_value(scales[oracle_tiled_scale_offset(r, b, cols)]);
            float res[16];
            float amax = 0.0f;
            for (size_t i = start; i < end; ++i) {
                uint8_t code = (i & 1) ? (uint8_t)(prow[i / 2] >> 4) : (uint8_t)(prow[i / 2] & 0x0f);
                res[i - start] = fmaf(-oracle_e2m1_value(code), sv, norm[r * cols + i]);
                amax = fmaxf(amax, fabsf(res[i - start]));
            }
            uint8_t sc = amax == 0.0f ? 0 : oracle_ue4m3_code(amax / 6.0f);
            float rs = oracle_e4m3_value(sc);
            residual_scales[oracle_tiled_scale_offset(r, b, cols)] = sc;
            for (size_t i = start; i < end; ++i) {
                uint8_t code = oracle_e2m1_code(rs == 0.0f ? 0.0f : res[i - start] / rs);
                if ((i & 1) == 0) rrow[i / 2] = code;
                else rrow[i / 2] |= (uint8_t)(code << 4);
            }
        }
    }
    free(norm);
}

/* Post-norm residual add followed by the quantizing pre-norm of the next block:
 * crates/eider-cuda/native/non_gemm.cu:746-870.  h = input * rsqrt(mean(input^2) + input_eps) * input_weight + residual
 * (the last multiply and the add contract to one FMA in the reference's build), written to `output`; then the RMSNorm
 * quantizer above on h with quant_weight / quant_eps / input_scale.  Sums of squares in double (see above). */
ORACLE_API void oracle_rms_norm_add_then_rms_norm_quantize_nvfp4(const float* input, const float* input_weight, const float* residual,
                                                                 float* output, const float* quant_weight, size_t rows, size_t cols,
                                                                 float input_eps, float quant_eps, float input_scale,
                                                                 uint8_t* packed, uint8_t* scales, float* norm_out) {
    for (size_t r = 0; r < rows; ++r) {
        const float* x = input + r * cols;
        double ss = 0.0;
        for (size_t i = 0; i < cols; ++i) ss += (double)x[i] * (double)x[i];
        float inv = 1.0f / sqrtf((float)ss / (float)cols + input_eps);
        for (size_t i = 0; i < cols; ++i) output[r * cols + i] = fmaf(x[i] * inv, input_weight[i], residual[r * cols + i]);
    }
    /* the quantizing norm tiles its scales with outer = row, exactly like the stand-alone producer */
    oracle_rms_norm_quantize_nvfp4(output, quant_weight, rows, cols, quant_eps, input_scale, packed, scales, norm_out);
}

/* Grouped W4A4 GEMM: per expert D_e[row][m] = alpha_e * sum_k X_e[row][k] * W_e[m][k], rounded to
 * bf16 (crates/eider-cuda/native/cutlass_grouped_gemm.cu:116-164; output [route][m],
 * non_gemm.cu:3080-3083).  Activations dequantised from the per-expert tiled scales. */
typedef struct { const uint8_t* act_packed; const uint8_t* act_scales; const uint32_t* offsets;
                 size_t scale_tile_bytes; const uint8_t* w_packed; const uint8_t* w_scales;
                 const float* alpha; size_t out_features, k; uint16_t* out; } gg_ctx;
static void gg_body(size_t eb, size_t ee, void* p) {
    gg_ctx* c = (gg_ctx*)p;
    size_t k = c->k, blocks = k / 16, nf = c->out_features;
    float* wde = (float*)malloc(nf * k * sizeof(float));
    float* arow = (float*)malloc(k * sizeof(float));
    for (size_t e = eb; e < ee; ++e) {
        size_t r0 = c->offsets[e], r1 = c->offsets[e + 1];
        if (r0 == r1) continue;
        size_t base = oracle_moe_scale_base((uint32_t)e, c->offsets, c->scale_tile_bytes);
        const uint8_t* wp = c->w_packed + e * nf * (k / 2);
        const uint8_t* ws = c->w_scales + e * nf * blocks;
        for (size_t m = 0; m < nf; ++m)
            for (size_t i = 0; i < k; ++i) {
                size_t flat = m * k + i;
                uint8_t nib = (flat & 1) ? (wp[flat / 2] >> 4) : (wp[flat / 2] & 0x0f);
                wde[flat] = oracle_e2m1_value(nib) * oracle_e4m3_value(ws[m * blocks + i / 16]);
            }
        for (size_t r = r0; r < r1; ++r) {
            for (size_t i = 0; i < k; ++i) {
                size_t flat = r * k + i;
                uint8_t nib = (flat & 1) ? (c->act_packed[flat / 2] >> 4) : (c->act_packed[flat / 2] & 0x0f);
                arow[i] = oracle_e2m1_value(nib) *
                          oracle_e4m3_value(c->act_scales[base + oracle_tiled_scale_offset(r - r0, i / 16, k)]);
            }
            for (size_t m = 0; m < nf; ++m) {
                float acc = 0.0f;
                const float* wr = wde + m * k;
                for (size_t i = 0; i < k; ++i) acc += arow[i] * wr[i];
                c->out[r * nf + m] = oracle_f32_to_bf16(acc * c->alpha[e]);
            }
        }
    }
    free(wde);
    free(arow);
}
ORACLE_API void oracle_moe_grouped_gemm(const uint8_t* act_packed, const uint8_t* act_scales,
                                        const uint32_t* offsets, size_t experts,
                                        size_t scale_tile_bytes, const uint8_t* w_packed,
                                        const uint8_t* w_scales_row_major, const float* alpha,
                                        size_t out_features, size_t k, uint16_t* out_bf16) {
    gg_ctx c = {act_packed, act_scales, offsets, scale_tile_bytes, w_packed, w_scales_row_major,
                alpha, out_features, k, out_bf16};
    parallel_for(experts, gg_body, &c);
}

/* Un-permute + weighted sum: crates/eider-cuda/native/non_gemm.cu:3735-3758, slot order. */
ORACLE_API void oracle_moe_combine(const uint32_t* route_to_sorted, const float* route_weights,
                                   const uint16_t* sorted_bf16, size_t rows, size_t len,
                                   size_t routes_per_row, float* out) {
    for (size_t r = 0; r < rows; ++r)
        for (size_t c = 0; c < len; ++c) {
            float sum = 0.0f;
            for (size_t s = 0; s < routes_per_row; ++s) {
                size_t route = r * routes_per_row + s;
                sum += oracle_bf16_to_f32(sorted_bf16[(size_t)route_to_sorted[route] * len + c]) *
                       route_weights[route];
            }
            out[r * len + c] = sum;
        }
}
