// Drop-in for launch_lm_head (src/launcher.s:2903-2970): file lm_head.cubin, entry lm_head,
// parameters (u64 weight, u64 input, u64 output), grid 62080 x 128 threads = 4 rows per CTA.
// weight fp16 [248320, 5120] row-major, input fp32 [5120], output fp32 [248320].  One warp per row,
// 128-bit streaming loads, fp32 accumulation in a fixed order.
#include <cuda_fp16.h>
#include <stdint.h>
#define LM_HIDDEN 5120
extern "C" __global__ void __launch_bounds__(128) lm_head(const __half* __restrict__ w, const float* __restrict__ x,
                                                          float* __restrict__ y) {
    __shared__ __align__(16) float xs[LM_HIDDEN];
    for (int i = threadIdx.x; i < LM_HIDDEN; i += blockDim.x) xs[i] = x[i];
    __syncthreads();
    const int lane = threadIdx.x & 31;
    const size_t row = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const uint4* wr = reinterpret_cast<const uint4*>(w + row * LM_HIDDEN);
    float a0 = 0.f, a1 = 0.f;
    for (int i = lane; i < LM_HIDDEN / 8; i += 32) {
        const uint4 v = __ldcs(wr + i);
        const uint32_t p[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&p[j]));
            a0 = fmaf(f.x, xs[i * 8 + 2 * j], a0);
            a1 = fmaf(f.y, xs[i * 8 + 2 * j + 1], a1);
        }
    }
    float t = a0 + a1;
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    if (lane == 0) y[row] = t;
}
