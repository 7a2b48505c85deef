// Drop-in for launch_activate (src/launcher.s:2074-2143): file activate.cubin, entry activate,
// parameters (u64 gate, u64 up, u64 out, u32 size), grid 68 x 256.  out = silu(gate) * up, the form
// the launcher and kernels.ls:61-66 describe (the shipped SASS computes gate * silu(up)); fp32.
#include <stdint.h>
extern "C" __global__ void activate(const float* __restrict__ gate, const float* __restrict__ up, float* __restrict__ out,
                                    uint32_t n) {
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        const float g = gate[i];
        out[i] = g / (1.0f + __expf(-g)) * up[i];
    }
}
