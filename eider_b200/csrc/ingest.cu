// Host-side weight ingest for the NVFP4 path: everything between a checkpoint's bytes and the image the kernels read.
// No device code and no CUDA call in this file; it is part of the same library so a binding links one object.
//
//   * Nvfp4Artifact   the reference's per-linear disk record, bit-compatible (crates/eider-format/src/nvfp4_artifact.rs:12-75:
//                     "EIDNVF4\0", version 1, 60-byte header, prefix, packed bytes, K16 scales)
//   * compressed-tensors globals are divisors: weight_scale_2 = 1 / weight_global_scale, input_scale = 1 / input_global_scale
//                     (crates/eider-format/src/modelopt.rs:480-519, 1137-1145)
//   * MXFP4 -> NVFP4  E8M0 K32 scales become two equal UE4M3 K16 scales when exactly representable (modelopt.rs:173-248)
//   * GGUF NVFP4      36-byte blocks (four scales + 32 split-half nibble bytes) -> adjacent nibbles, no decoding
//                     (crates/eider-format/src/gguf_nvfp4.rs:12-64)
//   * requantisation  f32 / bf16 / FP8 (per-tensor, per-channel, 128 x 128 E8M0 blocks) -> NVFP4 with unit global scale
//                     (modelopt.rs:524-716)
//   * prepared cache  "EIDB2P01": the packed bytes as they are plus the 128 x 4 tiled scales the tensor-core kernels read,
//                     so a restart skips the repack; the analogue of the reference's EIDW4A01 file
//                     (crates/eider-cuda/src/kernels/sm121_w4a16.rs:18-20, 146-240)
//
// Return codes: 0 ok, 1 shape error, 2 format error, 3 I/O error (the reference's Error::Shape / Error::Format kinds).
#include <cmath>
#include <cstdio>
#include <cstring>
#include <string>
#include <thread>
#include <vector>

#include <unistd.h>

#include "common.cuh"
#include "eider_b200.h"

namespace eider {
namespace {

enum : int { kOk = 0, kShape = 1, kFormat = 2, kIo = 3 };

constexpr char kArtifactMagic[8] = {'E', 'I', 'D', 'N', 'V', 'F', '4', '\0'};
constexpr uint32_t kArtifactVersion = 1;
constexpr uint64_t kArtifactHeader = 60;
constexpr char kCacheMagic[8] = {'E', 'I', 'D', 'B', '2', 'P', '0', '1'};
constexpr uint32_t kCacheVersion = 1;
constexpr uint64_t kCacheHeader = 48;

float e8m0_value(uint8_t code) {  // crates/eider-cuda/src/format.rs:112-119: 2^(code - 127), 255 = NaN
    if (code == 255) return NAN;
    return std::ldexp(1.0f, static_cast<int>(code) - 127);
}

// crates/eider-cuda/src/format.rs:151-167: nearest UE4M3 code, ties to the even code, saturating at 0x7e.
uint8_t ue4m3_code_host(float v) {
    if (!std::isfinite(v) || v <= 0.0f) return 0;
    uint8_t best = 0;
    float best_err = v;  // error of code 0
    for (int code = 1; code <= 0x7e; ++code) {
        const float err = std::fabs(e4m3_value(static_cast<uint8_t>(code)) - v);
        if (err < best_err || (err == best_err && (code & 1) == 0 && (best & 1) != 0)) {
            best_err = err;
            best = static_cast<uint8_t>(code);
        }
    }
    return best;
}

// crates/eider-cuda/src/format.rs:44-76: nearest E2M1 magnitude, ties to the even code, saturating, NaN -> 0x7.
uint8_t e2m1_code_host(float v) {
    if (std::isnan(v)) return 0x7;
    const uint8_t sign = std::signbit(v) ? 0x8 : 0x0;
    const float a = std::fabs(v);
    static const float mags[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};
    if (a > 6.0f) return sign | 7;
    uint8_t best = 0;
    float best_err = a;
    for (uint8_t c = 1; c < 8; ++c) {
        const float err = std::fabs(mags[c] - a);
        if (err < best_err || (err == best_err && (c & 1) == 0 && (best & 1) == 1)) {
            best_err = err;
            best = c;
        }
    }
    return sign | best;
}

float bf16_to_f32(uint16_t b) {
    const uint32_t bits = static_cast<uint32_t>(b) << 16;
    float f;
    std::memcpy(&f, &bits, 4);
    return f;
}

bool write_all(FILE* f, const void* p, size_t n) { return n == 0 || std::fwrite(p, 1, n, f) == n; }
bool read_all(FILE* f, void* p, size_t n) { return n == 0 || std::fread(p, 1, n, f) == n; }

struct TempFile {
    std::string tmp, final_path;
    FILE* f;
    explicit TempFile(const char* path) : tmp(std::string(path) + ".tmp-" + std::to_string(getpid())), final_path(path) {
        f = std::fopen(tmp.c_str(), "wb");
    }
    int commit(bool ok) {
        if (f) ok = (std::fflush(f) == 0) && ok, ok = (std::fclose(f) == 0) && ok;
        f = nullptr;
        if (!ok || std::rename(tmp.c_str(), final_path.c_str()) != 0) {
            std::remove(tmp.c_str());
            return kIo;
        }
        return kOk;
    }
};

long long file_size(FILE* f) {
    if (std::fseek(f, 0, SEEK_END) != 0) return -1;
    const long long n = std::ftell(f);
    std::rewind(f);
    return n;
}

int validate_artifact(const char* prefix, uint64_t prefix_len, uint64_t out_features, uint64_t in_features, uint64_t packed_len,
                      uint64_t scale_len, float weight_scale_2, float input_scale) {
    if (out_features == 0 || in_features == 0 || in_features % 16 != 0) return kShape;
    if (out_features > UINT64_MAX / in_features) return kShape;
    const uint64_t elements = out_features * in_features;
    if (packed_len != elements / 2 || scale_len != elements / 16) return kShape;
    if (!prefix || prefix_len == 0 || !std::isfinite(weight_scale_2) || !std::isfinite(input_scale)) return kFormat;
    return kOk;
}

// ModelOptNvfp4Linear::quantize_values (crates/eider-format/src/modelopt.rs:649-716): rows split over the host threads.
template <typename ValueAt>
void quantize_values(uint64_t out_features, uint64_t in_features, ValueAt value_at, uint8_t* packed, uint8_t* scales) {
    const uint64_t blocks_per_row = in_features / 16;
    unsigned workers = std::thread::hardware_concurrency();
    if (workers == 0) workers = 1;
    if (workers > out_features) workers = static_cast<unsigned>(out_features);
    const uint64_t rows_per = (out_features + workers - 1) / workers;
    std::vector<std::thread> pool;
    for (unsigned w = 0; w < workers; ++w) {
        const uint64_t r0 = w * rows_per, r1 = r0 + rows_per < out_features ? r0 + rows_per : out_features;
        if (r0 >= r1) break;
        pool.emplace_back([=] {
            for (uint64_t row = r0; row < r1; ++row) {
                for (uint64_t block = 0; block < blocks_per_row; ++block) {
                    const uint64_t start = row * in_features + block * 16;
                    float v[16];
                    float max_abs = 0.0f;
                    for (int i = 0; i < 16; ++i) {
                        v[i] = value_at(start + i);
                        if (std::isfinite(v[i])) max_abs = std::fmax(max_abs, std::fabs(v[i]));
                    }
                    const uint8_t code = max_abs != 0.0f ? ue4m3_code_host(max_abs / 6.0f) : 0;
                    const float s = e4m3_value(code);
                    scales[row * blocks_per_row + block] = code;
                    for (int i = 0; i < 16; i += 2) {
                        const uint8_t lo = e2m1_code_host(s == 0.0f ? 0.0f : v[i] / s);
                        const uint8_t hi = e2m1_code_host(s == 0.0f ? 0.0f : v[i + 1] / s);
                        packed[(start + i) / 2] = static_cast<uint8_t>(lo | (hi << 4));
                    }
                }
            }
        });
    }
    for (auto& t : pool) t.join();
}

}  // namespace
}  // namespace eider

using namespace eider;

extern "C" {

int eider_b200_nvfp4_artifact_write(const char* path, const char* prefix, uint64_t out_features, uint64_t in_features,
                                    const uint8_t* packed_weight, uint64_t packed_len, const uint8_t* weight_scale, uint64_t scale_len,
                                    float weight_scale_2, float input_scale) {
    if (!path || !packed_weight || !weight_scale) return kShape;
    const uint64_t prefix_len = prefix ? std::strlen(prefix) : 0;
    if (int st = validate_artifact(prefix, prefix_len, out_features, in_features, packed_len, scale_len, weight_scale_2, input_scale)) return st;
    TempFile t(path);
    if (!t.f) return kIo;
    const uint64_t fields[5] = {out_features, in_features, packed_len, scale_len, prefix_len};  // little-endian hosts only
    bool ok = write_all(t.f, kArtifactMagic, 8) && write_all(t.f, &kArtifactVersion, 4) && write_all(t.f, fields, sizeof(fields)) &&
              write_all(t.f, &weight_scale_2, 4) && write_all(t.f, &input_scale, 4) && write_all(t.f, prefix, prefix_len) &&
              write_all(t.f, packed_weight, packed_len) && write_all(t.f, weight_scale, scale_len);
    return t.commit(ok);
}

int eider_b200_nvfp4_artifact_read_header(const char* path, uint64_t* out_features, uint64_t* in_features, uint64_t* packed_len,
                                          uint64_t* scale_len, uint64_t* prefix_len, float* weight_scale_2, float* input_scale) {
    if (!path || !out_features || !in_features || !packed_len || !scale_len || !prefix_len || !weight_scale_2 || !input_scale)
        return kShape;
    FILE* f = std::fopen(path, "rb");
    if (!f) return kIo;
    const long long size = file_size(f);
    char magic[8];
    uint32_t version = 0;
    uint64_t fields[5];
    const bool ok = read_all(f, magic, 8) && read_all(f, &version, 4) && read_all(f, fields, sizeof(fields)) &&
                    read_all(f, weight_scale_2, 4) && read_all(f, input_scale, 4);
    std::fclose(f);
    if (!ok) return kIo;
    if (std::memcmp(magic, kArtifactMagic, 8) != 0 || version != kArtifactVersion) return kFormat;
    *out_features = fields[0];
    *in_features = fields[1];
    *packed_len = fields[2];
    *scale_len = fields[3];
    *prefix_len = fields[4];
    // the payload must be exactly what the header announces
    const uint64_t expected = kArtifactHeader + fields[4] + fields[2] + fields[3];
    if (expected < kArtifactHeader || size < 0 || static_cast<uint64_t>(size) != expected) return kFormat;
    return kOk;
}

int eider_b200_nvfp4_artifact_read(const char* path, char* prefix, uint64_t prefix_capacity, uint8_t* packed_weight,
                                   uint64_t packed_capacity, uint8_t* weight_scale, uint64_t scale_capacity) {
    uint64_t out_features, in_features, packed_len, scale_len, prefix_len;
    float w2, is;
    if (int st = eider_b200_nvfp4_artifact_read_header(path, &out_features, &in_features, &packed_len, &scale_len, &prefix_len, &w2, &is))
        return st;
    if (!prefix || !packed_weight || !weight_scale || prefix_capacity < prefix_len + 1 || packed_capacity < packed_len ||
        scale_capacity < scale_len)
        return kShape;
    FILE* f = std::fopen(path, "rb");
    if (!f) return kIo;
    bool ok = std::fseek(f, static_cast<long>(kArtifactHeader), SEEK_SET) == 0 && read_all(f, prefix, prefix_len) &&
              read_all(f, packed_weight, packed_len) && read_all(f, weight_scale, scale_len);
    std::fclose(f);
    if (!ok) return kIo;
    prefix[prefix_len] = '\0';
    return validate_artifact(prefix, prefix_len, out_features, in_features, packed_len, scale_len, w2, is);
}

int eider_b200_compressed_tensors_globals(float weight_global_scale, float input_global_scale, float* weight_scale_2,
                                          float* input_scale) {
    if (!weight_scale_2 || !input_scale) return kShape;
    if (!std::isfinite(weight_global_scale) || weight_global_scale <= 0.0f || !std::isfinite(input_global_scale) ||
        input_global_scale <= 0.0f)
        return kFormat;
    *weight_scale_2 = 1.0f / weight_global_scale;
    *input_scale = 1.0f / input_global_scale;
    return kOk;
}

int eider_b200_mxfp4_scales_to_nvfp4(const uint8_t* e8m0_scales, uint64_t count, uint8_t* ue4m3_scales) {
    if (!e8m0_scales || !ue4m3_scales) return kShape;
    for (uint64_t i = 0; i < count; ++i) {
        const float value = e8m0_value(e8m0_scales[i]);
        if (!std::isfinite(value)) return kFormat;
        const uint8_t code = ue4m3_code_host(value);
        if (e4m3_value(code) != value) return kFormat;  // outside the range UE4M3 holds exactly
        ue4m3_scales[2 * i] = code;
        ue4m3_scales[2 * i + 1] = code;
    }
    return kOk;
}

int eider_b200_gguf_nvfp4_unpack(const uint8_t* blocks, uint64_t bytes, uint64_t out_features, uint64_t in_features,
                                 float global_scale, uint8_t* packed_weight, uint8_t* weight_scale) {
    if (!blocks || !packed_weight || !weight_scale) return kShape;
    if (out_features == 0 || in_features == 0 || in_features % 64 != 0 || out_features > UINT64_MAX / in_features) return kFormat;
    const uint64_t elements = out_features * in_features;
    if (bytes != elements / 64 * 36 || !std::isfinite(global_scale) || global_scale <= 0.0f) return kFormat;
    for (uint64_t b = 0; b < elements / 64; ++b) {
        const uint8_t* block = blocks + b * 36;
        for (int i = 0; i < 4; ++i)
            if (block[i] >= 0x7f) return kFormat;  // UE4M3 has no sign and 0x7f is not finite
        std::memcpy(weight_scale + b * 4, block, 4);
        for (int group = 0; group < 4; ++group) {
            const uint8_t* src = block + 4 + group * 8;
            uint8_t* dst = packed_weight + b * 32 + group * 8;
            for (int j = 0; j < 4; ++j) {
                dst[j] = static_cast<uint8_t>((src[2 * j] & 15) | ((src[2 * j + 1] & 15) << 4));
                dst[j + 4] = static_cast<uint8_t>((src[2 * j] >> 4) | (src[2 * j + 1] & 0xf0));
            }
        }
    }
    return kOk;
}

int eider_b200_nvfp4_requantize_host(int source_kind, const void* values, const float* channel_scale, float tensor_scale,
                                     const uint8_t* block_scale_e8m0, uint64_t out_features, uint64_t in_features,
                                     uint8_t* packed_weight, uint8_t* weight_scale) {
    if (!values || !packed_weight || !weight_scale || out_features == 0 || in_features == 0 || in_features % 16 != 0) return kShape;
    switch (source_kind) {
        case 0: {  // f32
            const float* v = static_cast<const float*>(values);
            quantize_values(out_features, in_features, [=](uint64_t i) { return v[i]; }, packed_weight, weight_scale);
            return kOk;
        }
        case 1: {  // bf16 (modelopt.rs:524-545)
            const uint16_t* v = static_cast<const uint16_t*>(values);
            quantize_values(out_features, in_features, [=](uint64_t i) { return bf16_to_f32(v[i]); }, packed_weight, weight_scale);
            return kOk;
        }
        case 2: {  // FP8 E4M3 with a per-tensor or per-channel scale (modelopt.rs:547-592)
            if (!std::isfinite(tensor_scale)) return kFormat;
            if (channel_scale)
                for (uint64_t r = 0; r < out_features; ++r)
                    if (!std::isfinite(channel_scale[r])) return kShape;
            const uint8_t* v = static_cast<const uint8_t*>(values);
            quantize_values(out_features, in_features,
                            [=](uint64_t i) { return e4m3_value(v[i]) * (channel_scale ? channel_scale[i / in_features] : tensor_scale); },
                            packed_weight, weight_scale);
            return kOk;
        }
        case 3: {  // FP8 E4M3 with 128 x 128 E8M0 block scales (modelopt.rs:594-645)
            if (!block_scale_e8m0 || out_features % 128 != 0 || in_features % 128 != 0) return kShape;
            const uint64_t scale_cols = in_features / 128;
            for (uint64_t i = 0; i < (out_features / 128) * scale_cols; ++i)
                if (block_scale_e8m0[i] == 255) return kFormat;
            const uint8_t* v = static_cast<const uint8_t*>(values);
            quantize_values(out_features, in_features,
                            [=](uint64_t i) {
                                const uint64_t row = i / in_features, col = i % in_features;
                                return e4m3_value(v[i]) * e8m0_value(block_scale_e8m0[(row / 128) * scale_cols + col / 128]);
                            },
                            packed_weight, weight_scale);
            return kOk;
        }
        default: return kShape;
    }
}

void eider_b200_nvfp4_scales_to_tiled_host(const uint8_t* scales_row_major, uint8_t* scales_tiled, uint64_t out_features,
                                           uint64_t in_features) {
    // modelopt_scales_to_cublaslt (crates/eider-format/src/modelopt.rs:1148-1161); padding bytes are zero
    std::memset(scales_tiled, 0, scale_layout_len(out_features, in_features));
    const uint64_t blocks = in_features / 16;
    for (uint64_t o = 0; o < out_features; ++o)
        for (uint64_t b = 0; b < blocks; ++b)
            scales_tiled[tiled_scale_offset(static_cast<uint32_t>(o), static_cast<uint32_t>(b), static_cast<uint32_t>(in_features))] =
                scales_row_major[o * blocks + b];
}

int eider_b200_prepared_cache_write(const char* path, uint64_t out_features, uint64_t in_features, const uint8_t* packed_weight,
                                    const uint8_t* scales_tiled, float weight_scale_2) {
    if (!path || !packed_weight || !scales_tiled || out_features == 0 || in_features == 0 || in_features % 32 != 0) return kShape;
    if (!std::isfinite(weight_scale_2)) return kFormat;
    const uint64_t weight_bytes = out_features * in_features / 2, scale_bytes = scale_layout_len(out_features, in_features);
    TempFile t(path);
    if (!t.f) return kIo;
    const uint64_t fields[4] = {out_features, in_features, weight_bytes, scale_bytes};
    bool ok = write_all(t.f, kCacheMagic, 8) && write_all(t.f, &kCacheVersion, 4) && write_all(t.f, fields, sizeof(fields)) &&
              write_all(t.f, &weight_scale_2, 4) && write_all(t.f, packed_weight, weight_bytes) && write_all(t.f, scales_tiled, scale_bytes);
    return t.commit(ok);
}

int eider_b200_prepared_cache_matches(const char* path, uint64_t out_features, uint64_t in_features) {
    if (!path || out_features == 0 || in_features == 0 || in_features % 32 != 0) return 0;
    FILE* f = std::fopen(path, "rb");
    if (!f) return 0;
    const uint64_t weight_bytes = out_features * in_features / 2, scale_bytes = scale_layout_len(out_features, in_features);
    const long long size = file_size(f);
    char magic[8];
    uint32_t version = 0;
    uint64_t fields[4] = {0, 0, 0, 0};
    const bool ok = read_all(f, magic, 8) && read_all(f, &version, 4) && read_all(f, fields, sizeof(fields));
    std::fclose(f);
    return ok && size >= 0 && static_cast<uint64_t>(size) == kCacheHeader + weight_bytes + scale_bytes &&
           std::memcmp(magic, kCacheMagic, 8) == 0 && version == kCacheVersion && fields[0] == out_features && fields[1] == in_features &&
           fields[2] == weight_bytes && fields[3] == scale_bytes;
}

int eider_b200_prepared_cache_read(const char* path, uint64_t out_features, uint64_t in_features, uint8_t* packed_weight,
                                   uint8_t* scales_tiled, float* weight_scale_2) {
    if (!packed_weight || !scales_tiled || !weight_scale_2) return kShape;
    if (!eider_b200_prepared_cache_matches(path, out_features, in_features)) return kFormat;
    FILE* f = std::fopen(path, "rb");
    if (!f) return kIo;
    const uint64_t weight_bytes = out_features * in_features / 2, scale_bytes = scale_layout_len(out_features, in_features);
    const bool ok = std::fseek(f, static_cast<long>(kCacheHeader - 4), SEEK_SET) == 0 && read_all(f, weight_scale_2, 4) &&
                    read_all(f, packed_weight, weight_bytes) && read_all(f, scales_tiled, scale_bytes);
    std::fclose(f);
    if (!ok) return kIo;
    return std::isfinite(*weight_scale_2) ? kOk : kFormat;
}

}  // extern "C"
