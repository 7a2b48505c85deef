// Drop-in for launch_rope: file rotate.cubin.
//
// `rotate`: the launcher's 7-parameter block (src/launcher.s:2260-2267):
//   (u64 q, u64 k, u64 cos, u64 sin, u32 seq_pos, u32 head_dim, u32 num_heads), grid num_heads x head_dim threads,
// table-driven half-split rotation as launched: pair (i, i + head_dim/2), i < head_dim/2, with
// cos[seq_pos * head_dim/2 + i], sin[...] from the host tables (src/launcher.s:3139-3148: [32768][128] fp32).  q has
// num_heads heads; the launcher's k slice holds 4 KV heads (src/launcher.s:2157-2160: 4096 bytes), so k is rotated for
// head blocks < num_heads / 6 (the model's 24 : 4 grouping) -- the launcher's 24-block launch would otherwise run
// over the V slice that follows K.  In place, fp32.
//
// `rope`: the parameter block of inference/attend.ls:21-25 (u64 q, u64 k, u64 q_out, u64 k_out, u32 d_head, u32 pos),
// grid = heads x 128 pair lanes: interleaved pairs (2i, 2i+1) for i < 32 with frequency 2^(-23.25349666 i / 32)
// (theta 1e7), the other 96 pairs copied.  One block per head; k is rotated where k != 0 (pass 0 for a q-only launch).
// The angle is formed and reduced in double: at positions in the thousands a float32 product pos * freq has lost the
// bits the rotation needs.
#include <stdint.h>

extern "C" __global__ void __launch_bounds__(256) rotate(float* q, float* k, const float* cos_t, const float* sin_t, uint32_t seq_pos,
                                                         uint32_t head_dim, uint32_t num_heads) {
    const uint32_t h = blockIdx.x, i = threadIdx.x, half = head_dim / 2;
    if (h >= num_heads || i >= half) return;
    const float c = cos_t[(size_t)seq_pos * half + i], s = sin_t[(size_t)seq_pos * half + i];
    float* x = q + (size_t)h * head_dim;
    const float a = x[i], b = x[i + half];
    x[i] = a * c - b * s;
    x[i + half] = a * s + b * c;
    const uint32_t kv_heads = num_heads >= 6 ? num_heads / 6 : 1;
    if (h < kv_heads) {
        float* y = k + (size_t)h * head_dim;
        const float a2 = y[i], b2 = y[i + half];
        y[i] = a2 * c - b2 * s;
        y[i + half] = a2 * s + b2 * c;
    }
}

extern "C" __global__ void __launch_bounds__(128) rope(const float* q, const float* k, float* q_out, float* k_out, uint32_t d_head, uint32_t pos) {
    const uint32_t h = blockIdx.x, i = threadIdx.x;
    if (2 * i + 1 >= d_head) return;
    float c = 1.f, s = 0.f;
    if (i < 32) {
        const double a = (double)pos * exp2(-23.25349666421 * (double)i / 32.0);
        const double n = rint(a * 0.15915494309189535);
        sincosf((float)fma(-n, 6.283185307179586, a), &s, &c);
    }
    const size_t e = (size_t)h * d_head + 2 * i;
    const float q0 = q[e], q1 = q[e + 1];
    q_out[e] = q0 * c - q1 * s;
    q_out[e + 1] = q0 * s + q1 * c;
    if (k) {
        const float k0 = k[e], k1 = k[e + 1];
        k_out[e] = k0 * c - k1 * s;
        k_out[e + 1] = k0 * s + k1 * c;
    }
}
