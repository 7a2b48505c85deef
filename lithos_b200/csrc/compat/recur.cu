// Drop-in for launch_recurrence: file recur.cubin.
//
// Primary entry `deltanet_fused`: the parameter block of inference/deltanet_fused.ls:37-41
//   (u64 q, u64 k, u64 v, u64 z, u64 decay, u64 beta, u64 state, u64 output, u32 d, u32 gqa), grid = key heads (16), block d (128).
// All fp32.  q, k [key heads, 128]; v, z, output [key heads * gqa, 128]; decay, beta [key heads * gqa]; state
// [key heads, gqa, 128, 128] updated in place (row = key index, column = value index).  Per value head, as the text
// states it (deltanet_fused.ls:97-149): r = S^T k from the OLD, un-decayed state; delta = beta (v - r);
// S = decay S + k delta^T; out = S_new^T q; out *= silu(z).  Thread j owns column j of the state.
//
// `deltanet_step`: the entry name the launcher resolves in recur.cubin, with ITS 7-parameter block
// (src/launcher.s:1960-1968): (u64 state, u64 query, u64 unused, u64 key, u64 value, u64 output, u32 count), grid
// ceil(count / 256) x 256, element-wise state[i] += value[i] * key[i]; output[i] = query[i] * state[i] -- the
// placeholder arithmetic the launcher documents (inference/recur.ls:61-78), kept so that the launcher's own call
// sequence runs unchanged; the model's recurrence is `deltanet_fused`.
#include <stdint.h>

extern "C" __global__ void __launch_bounds__(128) deltanet_fused(const float* __restrict__ q, const float* __restrict__ k,
                                                                 const float* __restrict__ v, const float* __restrict__ z,
                                                                 const float* __restrict__ decay, const float* __restrict__ beta,
                                                                 float* __restrict__ state, float* __restrict__ output, uint32_t d, uint32_t gqa) {
    __shared__ float sk[128], sq[128];
    const int kh = blockIdx.x, j = threadIdx.x;
    if (d != 128 || blockDim.x != 128) return;
    sk[j] = k[(size_t)kh * 128 + j];
    sq[j] = q[(size_t)kh * 128 + j];
    __syncthreads();
    for (uint32_t vo = 0; vo < gqa; ++vo) {
        const size_t vh = (size_t)kh * gqa + vo;
        float* S = state + vh * 128 * 128;
        const float g = decay[vh], b = beta[vh];
        // pass 1: column j of the old state against k (128 coalesced row reads, four independent chains)
        float r0 = 0.f, r1 = 0.f, r2 = 0.f, r3 = 0.f;
        for (int i = 0; i < 128; i += 4) {
            r0 = fmaf(sk[i], S[(size_t)i * 128 + j], r0);
            r1 = fmaf(sk[i + 1], S[(size_t)(i + 1) * 128 + j], r1);
            r2 = fmaf(sk[i + 2], S[(size_t)(i + 2) * 128 + j], r2);
            r3 = fmaf(sk[i + 3], S[(size_t)(i + 3) * 128 + j], r3);
        }
        const float delta = b * (v[vh * 128 + j] - ((r0 + r1) + (r2 + r3)));
        // pass 2: decay, rank-one update, read-out from the new state
        float a0 = 0.f, a1 = 0.f;
        for (int i = 0; i < 128; i += 2) {
            const float s0 = fmaf(sk[i], delta, g * S[(size_t)i * 128 + j]);
            const float s1 = fmaf(sk[i + 1], delta, g * S[(size_t)(i + 1) * 128 + j]);
            S[(size_t)i * 128 + j] = s0;
            S[(size_t)(i + 1) * 128 + j] = s1;
            a0 = fmaf(s0, sq[i], a0);
            a1 = fmaf(s1, sq[i + 1], a1);
        }
        const float zz = z[vh * 128 + j];
        output[vh * 128 + j] = (a0 + a1) * (zz / (1.0f + __expf(-zz)));
    }
}

extern "C" __global__ void deltanet_step(float* __restrict__ state, const float* __restrict__ query, const void* unused,
                                         const float* __restrict__ key, const float* __restrict__ value, float* __restrict__ output,
                                         uint32_t count) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= count) return;
    const float s = fmaf(value[i], key[i], state[i]);
    state[i] = s;
    output[i] = query[i] * s;
}
