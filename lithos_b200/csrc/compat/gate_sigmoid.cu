// Drop-in for launch_gate_sigmoid (src/launcher.s:2459-2533): file gate_sigmoid.cubin, entry
// gate_sigmoid, parameters (u64 output, u64 z, u32 n), grid 24 x 256.  output[i] *= sigmoid(z[i]); fp32.
#include <stdint.h>
extern "C" __global__ void gate_sigmoid(float* __restrict__ out, const float* __restrict__ z, uint32_t n) {
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x)
        out[i] *= 1.0f / (1.0f + __expf(-z[i]));
}
