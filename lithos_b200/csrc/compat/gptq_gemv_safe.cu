// Drop-in for the reference's launched GEMV: same file name, entry name,
// parameter block, launch geometry and arithmetic as minds/gptq_gemv_safe.ptx
// (parameter block :46-55; launch grid (ceil(N/256), K_SPLITS), block 64,
// dynamic shared memory 4*K bytes, src/launcher.s:1479-1535), rebuilt for
// sm_100a.
//
//   y[n] += sum_k fma(float(q), s, -8 s) * x[k]      x, y fp32; zero-point 8
//
// Per column the products are accumulated with fp32 FMAs in ascending k, the
// order the reference kernel uses, so with K_SPLITS == 1 the result is
// bit-identical to the reference's; the split partials are combined with
// atomicAdd exactly as there (the caller zeroes y).  What changes is the memory
// pipeline: one 128-bit load per packed row and 16 rows in flight per thread
// instead of four dependent 32-bit loads.
#include <cuda_fp16.h>
#include <stdint.h>

#define ROWS_IN_FLIGHT 16

__device__ __forceinline__ float nib_to_f32(uint32_t w, int j) {
    // exact int -> float without I2F: 2^23 + q, minus 2^23
    return __uint_as_float(0x4B000000u | ((w >> (4 * j)) & 0xFu)) - 8388608.0f;
}

__device__ __forceinline__ void fma_word(uint32_t w, float s, float b, const float* __restrict__ xs, float& acc) {
#pragma unroll
    for (int j = 0; j < 8; ++j) acc = fmaf(fmaf(nib_to_f32(w, j), s, b), xs[j], acc);
}

extern "C" __global__ void __launch_bounds__(64) gptq_gemv_safe(const uint32_t* __restrict__ qweight,
                                                               const __half* __restrict__ scales,
                                                               const float* __restrict__ x, float* __restrict__ y,
                                                               uint32_t N, uint32_t K, uint32_t K_SPLITS,
                                                               uint32_t k_packed_per_split) {
    extern __shared__ __align__(16) float xs[];
    const uint32_t col0 = blockIdx.x * 256u + threadIdx.x * 4u;
    const uint32_t kp_total = K >> 3;
    const uint32_t kp0 = min(blockIdx.y * k_packed_per_split, kp_total);
    const uint32_t kp1 = min(kp0 + k_packed_per_split, kp_total);
    if (kp1 == kp0) return;
    (void)K_SPLITS;
    for (uint32_t i = threadIdx.x; i < (kp1 - kp0) * 8u; i += blockDim.x) xs[i] = x[kp0 * 8u + i];
    __syncthreads();
    if (col0 >= N) return;
    const bool full = col0 + 3u < N; // all four columns valid: 128-bit loads
    float acc[4] = {0.f, 0.f, 0.f, 0.f}, s[4] = {0.f, 0.f, 0.f, 0.f}, b[4] = {0.f, 0.f, 0.f, 0.f};
    uint32_t cur_group = 0xffffffffu;
    for (uint32_t kp = kp0; kp < kp1; kp += ROWS_IN_FLIGHT) {
        uint4 w[ROWS_IN_FLIGHT];
#pragma unroll
        for (int r = 0; r < ROWS_IN_FLIGHT; ++r) {
            w[r] = make_uint4(0u, 0u, 0u, 0u);
            if (kp + r < kp1) {
                const uint32_t* p = qweight + (size_t)(kp + r) * N + col0;
                if (full) w[r] = __ldcs(reinterpret_cast<const uint4*>(p));
                else {
                    w[r].x = p[0];
                    if (col0 + 1u < N) w[r].y = p[1];
                    if (col0 + 2u < N) w[r].z = p[2];
                }
            }
        }
#pragma unroll
        for (int r = 0; r < ROWS_IN_FLIGHT; ++r) {
            if (kp + r < kp1) {
                const uint32_t g = (kp + r) >> 4;
                if (g != cur_group) {
                    cur_group = g;
#pragma unroll
                    for (int c = 0; c < 4; ++c)
                        if (col0 + c < N) {
                            s[c] = __half2float(scales[(size_t)g * N + col0 + c]);
                            b[c] = s[c] * -8.0f;
                        }
                }
                const float* xr = xs + (kp + r - kp0) * 8u;
                fma_word(w[r].x, s[0], b[0], xr, acc[0]);
                fma_word(w[r].y, s[1], b[1], xr, acc[1]);
                fma_word(w[r].z, s[2], b[2], xr, acc[2]);
                fma_word(w[r].w, s[3], b[3], xr, acc[3]);
            }
        }
    }
#pragma unroll
    for (int c = 0; c < 4; ++c)
        if (col0 + c < N) atomicAdd(y + col0 + c, acc[c]);
}
