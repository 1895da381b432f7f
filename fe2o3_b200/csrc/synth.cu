// Deterministic synthetic inputs, generated on the host.
//
// Element i of stream (seed, domain) is a pure function of (seed, domain, i):
// u = mix64(seed ^ mix64(domain) ^ i * odd_constant), the SplitMix64 finaliser the
// reference's generator uses (examples/tiled_gemm_v1/src/inputs.rs:54-79).
#include <math.h>
#include <string.h>
#include <stdint.h>

#include "common.cuh"

namespace {

inline uint64_t mix64(uint64_t v) {
    v += 0x9e3779b97f4a7c15ull;
    v = (v ^ (v >> 30)) * 0xbf58476d1ce4e5b9ull;
    v = (v ^ (v >> 27)) * 0x94d049bb133111ebull;
    return v ^ (v >> 31);
}
inline uint64_t rotl64(uint64_t v, unsigned r) { return (v << r) | (v >> (64 - r)); }
inline uint64_t draw(uint64_t key, uint64_t i) { return mix64(key ^ (i * 0xd6e8feb86659fd93ull)); }
inline uint64_t stream_key(uint64_t seed, uint64_t domain) { return seed ^ mix64(domain); }

inline float uniform_pm1(uint64_t u) { return (float)(u >> 40) * (1.0f / 8388608.0f) - 1.0f; }

// Box-Muller in f64 on two independent draws of the same index.
inline double normal01(uint64_t key, uint64_t i) {
    const uint64_t u1 = draw(key, 2 * i), u2 = draw(key, 2 * i + 1);
    const double a = ((double)(u1 >> 11) + 1.0) * (1.0 / 9007199254740992.0);  // (0, 1]
    const double b = (double)(u2 >> 11) * (1.0 / 9007199254740992.0);          // [0, 1)
    return sqrt(-2.0 * log(a)) * cos(6.283185307179586476925 * b);
}

}  // namespace

extern "C" {

uint16_t fe2o3_bf16_from_f32(float value) {
    uint32_t bits;
    memcpy(&bits, &value, 4);
    if ((bits & 0x7f800000u) == 0x7f800000u && (bits & 0x007fffffu) != 0) return (uint16_t)((bits >> 16) | 0x0040u);
    const uint32_t lsb = (bits >> 16) & 1u;
    return (uint16_t)((bits + 0x7fffu + lsb) >> 16);
}

int32_t fe2o3_synth_uniform_f32(uint64_t seed, uint64_t domain, uint64_t n, float *out) {
    const uint64_t key = stream_key(seed, domain);
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < (int64_t)n; ++i) out[i] = uniform_pm1(draw(key, (uint64_t)i));
    return FE2O3_OK;
}

int32_t fe2o3_synth_uniform_bf16(uint64_t seed, uint64_t domain, uint64_t n, uint16_t *out) {
    const uint64_t key = stream_key(seed, domain);
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < (int64_t)n; ++i) out[i] = fe2o3_bf16_from_f32(uniform_pm1(draw(key, (uint64_t)i)));
    return FE2O3_OK;
}

int32_t fe2o3_synth_normal_f32(uint64_t seed, uint64_t domain, uint64_t n, float sigma, float *out) {
    const uint64_t key = stream_key(seed, domain);
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < (int64_t)n; ++i) out[i] = (float)((double)sigma * normal01(key, (uint64_t)i));
    return FE2O3_OK;
}

int32_t fe2o3_synth_normal_bf16(uint64_t seed, uint64_t domain, uint64_t n, float sigma, uint16_t *out) {
    const uint64_t key = stream_key(seed, domain);
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < (int64_t)n; ++i)
        out[i] = fe2o3_bf16_from_f32((float)((double)sigma * normal01(key, (uint64_t)i)));
    return FE2O3_OK;
}

int32_t fe2o3_synth_u32_below(uint64_t seed, uint64_t domain, uint64_t n, uint32_t bound, uint32_t *out) {
    if (bound == 0) return FE2O3_ERR_INVALID_ARGUMENT;
    const uint64_t key = stream_key(seed, domain);
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < (int64_t)n; ++i)
        out[i] = (uint32_t)(((draw(key, (uint64_t)i) >> 32) * (uint64_t)bound) >> 32);
    return FE2O3_OK;
}

int32_t fe2o3_synth_bernoulli(uint64_t seed, uint64_t domain, uint64_t n, double p, uint32_t flag_value,
                              uint32_t *flags, uint64_t *packed) {
    if (!(p >= 0.0 && p <= 1.0)) return FE2O3_ERR_INVALID_ARGUMENT;
    const uint64_t key = stream_key(seed, domain);
    const uint64_t threshold = (uint64_t)(p * 4294967296.0);
    const uint64_t words = (n + 63) / 64;
#pragma omp parallel for schedule(static)
    for (int64_t w = 0; w < (int64_t)words; ++w) {
        uint64_t bits = 0;
        const uint64_t base = (uint64_t)w * 64;
        for (uint64_t l = 0; l < 64 && base + l < n; ++l) {
            const bool on = (draw(key, base + l) >> 32) < threshold;
            if (on) bits |= 1ull << l;
            if (flags) flags[base + l] = on ? flag_value : 0u;
        }
        if (packed) packed[w] = bits;
    }
    return FE2O3_OK;
}

int32_t fe2o3_synth_gemm_inputs_v1(uint32_t m, uint32_t n, uint32_t k, uint64_t seed, uint16_t *a_bits,
                                   uint16_t *b_bits) {
    static const uint16_t alphabet[16] = {0x0000, 0x3d80, 0xbd80, 0x3e00, 0xbe00, 0x3e80, 0xbe80, 0x3f00,
                                          0xbf00, 0x3f80, 0xbf80, 0x4000, 0xc000, 0x4040, 0xc040, 0x4080};
    const uint64_t shape_id = mix64((uint64_t)m ^ rotl64((uint64_t)n, 21) ^ rotl64((uint64_t)k, 42));
    const uint64_t ka = seed ^ shape_id ^ 0x5d7a91c431e2b80full, kb = seed ^ shape_id ^ 0xa2c56e3bce1d47f0ull;
    const uint64_t a_len = (uint64_t)m * k, b_len = (uint64_t)k * n;
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < (int64_t)a_len; ++i) a_bits[i] = alphabet[draw(ka, (uint64_t)i) % 16];
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < (int64_t)b_len; ++i) b_bits[i] = alphabet[draw(kb, (uint64_t)i) % 16];
    return FE2O3_OK;
}

}  // extern "C"
