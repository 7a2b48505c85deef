// Drop-in for the reference's sampling kernel (kernels/README.md:104-117, kernels/sample.sass): file
// sample.cubin, entry sample, parameters (u64 logits_f32, u64 output_token_u32, u32 vocab_size,
// f32 temperature, u32 top_k), grid 1 x 256.  The reference kernel scales every logit by 1/temperature
// and takes the arg-max with a strict ">" (inference/reduce.ls:214-313); it reads top_k and never
// uses it.  Same here, with the tie rule of the launcher's own CPU loop (src/launcher.s:1060-1063):
// the first maximum wins.  temperature <= 0 is taken as 1.  Only block 0 works, whatever the grid.
#include <stdint.h>
extern "C" __global__ void __launch_bounds__(1024) sample(const float* logits, uint32_t* out_token, uint32_t vocab, float temperature,
                                                          uint32_t top_k) {
    __shared__ float s_val[32];
    __shared__ uint32_t s_idx[32];
    if (blockIdx.x != 0) return;
    (void)top_k;
    const float inv_t = temperature > 0.f ? 1.0f / temperature : 1.0f;
    float best = -3.402823466e38f;
    uint32_t idx = 0xffffffffu;
    for (uint32_t i = threadIdx.x; i < vocab; i += blockDim.x) {
        const float v = logits[i] * inv_t;
        if (v > best) { best = v; idx = i; } // ascending i per thread: the first maximum stays
    }
    // (value, index) pairs: larger value wins, equal values keep the smaller index
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const uint32_t oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (ov > best || (ov == best && oi < idx)) { best = ov; idx = oi; }
    }
    if ((threadIdx.x & 31) == 0) { s_val[threadIdx.x >> 5] = best; s_idx[threadIdx.x >> 5] = idx; }
    __syncthreads();
    if (threadIdx.x < 32) {
        const uint32_t warps = (blockDim.x + 31) >> 5;
        best = threadIdx.x < warps ? s_val[threadIdx.x] : -3.402823466e38f;
        idx = threadIdx.x < warps ? s_idx[threadIdx.x] : 0xffffffffu;
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const uint32_t oi = __shfl_xor_sync(0xffffffffu, idx, o);
            if (ov > best || (ov == best && oi < idx)) { best = ov; idx = oi; }
        }
        if (threadIdx.x == 0) *out_token = idx == 0xffffffffu ? 0u : idx;
    }
}
