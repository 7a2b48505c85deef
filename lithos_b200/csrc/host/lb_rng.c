/* Seeded synthetic-tensor generator (host side, C).
 *
 * The model checkpoint and prompt the reference was measured with are not
 * distributable, so every tensor on the decode path is drawn from one 64-bit
 * seed with a counter-based generator: element i of stream s is a pure
 * function of (seed, s, i).  Any caller (this library's synthetic model
 * builder, the parity tests, the benchmark) that asks for the same
 * (seed, stream, count) gets bit-identical data, in any order and from any
 * number of threads.
 *
 * Distributions follow the reference's tensor formats:
 *   - qweight / qzeros: int32 words of 8 nibbles, each U{0..15}
 *     (GPTQ packing, minds/gptq_gemv_safe.ptx:46-55 parameter block);
 *   - scales: fp16  |N(0,1)|*0.01 + 1e-3;
 *   - activations / embeddings / norm weights: N(mean, std) rounded to
 *     fp16, bf16 or kept fp32.
 */
#include "lb_internal.h"
#include <math.h>

static inline uint64_t mix64(uint64_t z) {
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

uint64_t lb_rng_u64(uint64_t seed, uint64_t stream, uint64_t i) {
    uint64_t h = mix64(seed + 0x9E3779B97F4A7C15ull * (mix64(stream ^ 0xD1342543DE82EF95ull) | 1ull));
    return mix64(h + 0x9E3779B97F4A7C15ull * (i + 1));
}

/* uniform in (0,1), 24-bit resolution, never 0 or 1 */
static inline float u01(uint32_t bits) { return ((float)(bits >> 8) + 0.5f) * (1.0f / 16777216.0f); }

/* one standard normal per index (Box-Muller, cosine branch only) */
static inline float normal_at(uint64_t seed, uint64_t stream, uint64_t i) {
    uint64_t r = lb_rng_u64(seed, stream, i);
    float u1 = u01((uint32_t)(r >> 32)), u2 = u01((uint32_t)r);
    return sqrtf(-2.0f * logf(u1)) * cosf(6.28318530717958647692f * u2);
}

uint16_t lb_f32_to_f16(float f) {
    _Float16 h = (_Float16)f;
    uint16_t u;
    memcpy(&u, &h, 2);
    return u;
}
float lb_f16_to_f32(uint16_t u) {
    _Float16 h;
    memcpy(&h, &u, 2);
    return (float)h;
}
uint16_t lb_f32_to_bf16(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40); /* NaN */
    u += 0x7fffu + ((u >> 16) & 1u);                                          /* RNE */
    return (uint16_t)(u >> 16);
}
float lb_bf16_to_f32(uint16_t b) {
    uint32_t u = (uint32_t)b << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

/* single elements of the streams lb_fill_u32 / lb_fill_scales_f16 produce (the synthetic model builder draws only the
 * elements of its own tensor-parallel shard) */
uint32_t lb_rng_word(uint64_t seed, uint64_t stream, uint64_t i) { return (uint32_t)(lb_rng_u64(seed, stream, i) >> 32); }
uint16_t lb_rng_scale_f16(uint64_t seed, uint64_t stream, uint64_t i) {
    return lb_f32_to_f16(fabsf(normal_at(seed, stream, i)) * 0.01f + 1e-3f);
}

LB_API void lb_fill_u32(uint32_t* dst, size_t n, uint64_t seed, uint64_t stream) {
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < n; i++) dst[i] = (uint32_t)(lb_rng_u64(seed, stream, i) >> 32);
}

LB_API void lb_fill_normal_f32(float* dst, size_t n, uint64_t seed, uint64_t stream, float mean, float std) {
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < n; i++) dst[i] = mean + std * normal_at(seed, stream, i);
}

LB_API void lb_fill_normal_f16(uint16_t* dst, size_t n, uint64_t seed, uint64_t stream, float mean, float std) {
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < n; i++) dst[i] = lb_f32_to_f16(mean + std * normal_at(seed, stream, i));
}

LB_API void lb_fill_normal_bf16(uint16_t* dst, size_t n, uint64_t seed, uint64_t stream, float mean, float std) {
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < n; i++) dst[i] = lb_f32_to_bf16(mean + std * normal_at(seed, stream, i));
}

LB_API void lb_fill_uniform_f32(float* dst, size_t n, uint64_t seed, uint64_t stream, float lo, float hi) {
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < n; i++) dst[i] = lo + (hi - lo) * u01((uint32_t)(lb_rng_u64(seed, stream, i) >> 32));
}

/* GPTQ group scales: |N(0,1)|*0.01 + 1e-3, fp16 */
LB_API void lb_fill_scales_f16(uint16_t* dst, size_t n, uint64_t seed, uint64_t stream) {
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < n; i++) dst[i] = lb_f32_to_f16(fabsf(normal_at(seed, stream, i)) * 0.01f + 1e-3f);
}

LB_API void lb_convert_f32_to_f16(const float* src, uint16_t* dst, size_t n) {
    for (size_t i = 0; i < n; i++) dst[i] = lb_f32_to_f16(src[i]);
}
LB_API void lb_convert_f32_to_bf16(const float* src, uint16_t* dst, size_t n) {
    for (size_t i = 0; i < n; i++) dst[i] = lb_f32_to_bf16(src[i]);
}
LB_API void lb_convert_f16_to_f32(const uint16_t* src, float* dst, size_t n) {
    for (size_t i = 0; i < n; i++) dst[i] = lb_f16_to_f32(src[i]);
}
LB_API void lb_convert_bf16_to_f32(const uint16_t* src, float* dst, size_t n) {
    for (size_t i = 0; i < n; i++) dst[i] = lb_bf16_to_f32(src[i]);
}
