// Pieces shared by the decode-attention kernels: input loads, the per-head norm + partial RoPE of one 256-wide
// head vector, record layout of the slice partials.
#pragma once
#include "common.cuh"
#include "params.h"

#define AT_D 256
#define AT_THREADS 256
#define AT_WARPS 8
#define AT_GMAX 8
#define AT_REC 260 // floats per (kv, split, g) record: 256 acc + m + l + pad

__device__ __forceinline__ float ld_in(const void* p, size_t i, int is_f32) {
    return is_f32 ? reinterpret_cast<const float*>(p)[i]
                  : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
}

// One warp prepares one 256-wide head vector: RMS-normalise (plain weight), rotate the first
// rot_dims dims in interleaved pairs with the CTA's cos/sin table, scale, store to shared memory.
// A lane owns 8 consecutive dims, i.e. 4 rotation pairs.
__device__ __forceinline__ void warp_norm_rope(const void* src, size_t base, int is_f32, const uint16_t* w, float* dst,
                                               const float* cs_s, const float* sn_s, int rot_dims, float eps,
                                               float post_scale) {
    const int lane = threadIdx.x & 31;
    float v[8];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        v[j] = ld_in(src, base + lane * 8 + j, is_f32);
        ss += v[j] * v[j];
    }
    if (w) {
        ss = warp_sum(ss);
        const float r = rsqrtf(ss * (1.0f / AT_D) + eps);
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = v[j] * r * bf16_bits_to_f32(w[lane * 8 + j]);
    }
    if (lane * 8 < rot_dims) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int i = lane * 4 + j;
            if (2 * i < rot_dims) {
                const float a = v[2 * j], b = v[2 * j + 1], cs = cs_s[i], sn = sn_s[i];
                v[2 * j] = a * cs - b * sn;
                v[2 * j + 1] = a * sn + b * cs;
            }
        }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) dst[lane * 8 + j] = v[j] * post_scale;
}

