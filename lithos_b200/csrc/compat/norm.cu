// Drop-in for launch_norm (src/launcher.s:1101-1219): file norm.cubin, entry norm, parameters
// (u64 input, u64 residual, u64 weight, u64 output, u32 hidden_dim, f32 epsilon), grid = rows,
// block 256.  y = (x + r) * w * rsqrt(mean((x+r)^2) + eps) with the plain weight, as the shipped
// kernel and inference/reduce.ls:85-147 compute it; activations fp32, weight bf16 (the launcher
// hands over the checkpoint tensor, src/launcher.s:140-141).
#include <stdint.h>
// "norm" is also a CUDA math function with C linkage: the build renames compat_entry_norm to norm.
extern "C" __global__ void __launch_bounds__(256) compat_entry_norm(const float* __restrict__ x, const float* __restrict__ res,
                                                       const uint16_t* __restrict__ w, float* __restrict__ y,
                                                       uint32_t D, float eps) {
    __shared__ float red[33];
    const size_t row = (size_t)blockIdx.x * D;
    float ss = 0.f;
    for (uint32_t i = threadIdx.x; i < D; i += blockDim.x) {
        const float v = x[row + i] + (res ? res[row + i] : 0.f);
        ss += v * v;
    }
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x < 32) {
        float t = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
        for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
        if (threadIdx.x == 0) red[32] = rsqrtf(t / (float)D + eps);
    }
    __syncthreads();
    const float rinv = red[32];
    for (uint32_t i = threadIdx.x; i < D; i += blockDim.x) {
        const float v = x[row + i] + (res ? res[row + i] : 0.f);
        y[row + i] = v * rinv * __uint_as_float((uint32_t)w[i] << 16);
    }
}
