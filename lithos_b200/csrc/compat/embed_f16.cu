// Drop-in for the launcher's embed launch (src/launcher.s:713-762): file embed_f16.cubin, entry
// embed_f16, parameters (u32 token_id, u64 table, u64 out), grid 5 x 256 threads = 1280 threads,
// 4 elements each = the 5120-wide row.  Table fp16 [vocab, 5120] (inference/embed.ls:16-24), out fp32.
#include <cuda_fp16.h>
#include <stdint.h>
extern "C" __global__ void embed_f16(uint32_t token_id, const __half* __restrict__ table, float* __restrict__ out) {
    const uint32_t hidden = gridDim.x * blockDim.x * 4u;
    const uint32_t i = (blockIdx.x * blockDim.x + threadIdx.x) * 4u;
    const uint2 raw = *reinterpret_cast<const uint2*>(table + (size_t)token_id * hidden + i);
    const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&raw.x));
    const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&raw.y));
    *reinterpret_cast<float4*>(out + i) = make_float4(a.x, a.y, b.x, b.y);
}
