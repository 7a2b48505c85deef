// Drop-in for launch_l2norm (src/launcher.s:2366-2444): file reduce.cubin, entry l2norm, parameters
// (u64 x, u64 y, u32 hidden_dim), grid 1 x 256.  y = x * rsqrt(sum x^2), no epsilon
// (inference/reduce.ls:153-207), over the whole vector as launched; in place is allowed; fp32.
#include <stdint.h>
extern "C" __global__ void __launch_bounds__(256) l2norm(const float* x, float* y, uint32_t D) {
    __shared__ float red[33];
    const size_t row = (size_t)blockIdx.x * D;
    float ss = 0.f;
    for (uint32_t i = threadIdx.x; i < D; i += blockDim.x) ss += x[row + i] * x[row + i];
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x < 32) {
        float t = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
        for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
        if (threadIdx.x == 0) red[32] = rsqrtf(t);
    }
    __syncthreads();
    const float r = red[32];
    for (uint32_t i = threadIdx.x; i < D; i += blockDim.x) y[row + i] = x[row + i] * r;
}
