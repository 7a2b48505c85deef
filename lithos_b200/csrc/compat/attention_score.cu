// Drop-in for launch_attention: file attention_score.cubin.
//
// Primary entry `attention_score`: the parameter block of inference/attend.ls:85-90 (pointers first, then the
// `param` scalars in declaration order, bootstrap-py/codegen.py:372-377):
//   (u64 q, u64 k_cache, u64 v_cache, u64 output, u32 d_head, u32 seq_len, u32 current_pos, u32 n_kv_heads, u32 n_q_heads)
// grid = n_q_heads blocks of d_head (256) threads.  q [n_q_heads, 256] fp32 (already normalised and rotated), caches
// [position][n_kv_heads][256] (attend.ls:135-138), output [n_q_heads, 256] fp32.  Positions t < min(seq_len, current_pos)
// are attended (attend.ls:127-131), query head h reads KV head h * n_kv_heads / n_q_heads (attend.ls:101-104), scores are
// scaled by rsqrt(d_head).  Soft-max with the natural exponential and a true -inf start (attend_full.ls:186-196); the
// attend.ls text's 2^x without the log2(e) factor and its running maximum starting at -8 (attend.ls:119,168-176) are
// not reproduced.  `attention_score` reads an fp32 cache (the .ls arrays and the launcher's cache are fp32),
// `attention_score_bf16` the bf16 cache this library's own decode step keeps.
//
// `attention_score_launcher`: the 7-parameter block the launcher builds (src/launcher.s:1846-1853):
//   (u64 q, u64 k_cache, u64 v_cache, u64 output, u32 seq_len, u32 head_dim, u32 num_heads), grid 24 x 256,
// fp32 cache rows of 4 KV heads x 256 (src/launcher.s:2162-2166: 4096 bytes per position), positions t < seq_len, GQA
// map as above with n_kv_heads = 4.  (A cubin cannot hold two entries of one name, so a maintainer who keeps the
// launcher's block points kname_attn at this symbol.)
#include <cuda_bf16.h>
#include <stdint.h>

template <typename T> __device__ __forceinline__ float ld_kv(const T* p, size_t i);
template <> __device__ __forceinline__ float ld_kv<float>(const float* p, size_t i) { return p[i]; }
template <> __device__ __forceinline__ float ld_kv<__nv_bfloat16>(const __nv_bfloat16* p, size_t i) { return __bfloat162float(p[i]); }

// One CTA per query head, 8 warps; warp w takes positions w, w+8, ...; a lane owns 8 of the 256 dims.  Online soft-max
// per warp, the 8 warps merged through shared memory in warp order (fixed order: run-to-run identical bits).
template <typename T>
__device__ __forceinline__ void attention_core(const float* q, const T* kc, const T* vc, float* out, int L, int n_kv, int n_q) {
    constexpr int D = 256, W = 8;
    __shared__ float s_m[W], s_l[W], s_acc[W][D];
    const int h = blockIdx.x, lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    if (h >= n_q || blockDim.x != D) return;
    const int kv = (int)((long long)h * n_kv / n_q);
    float qv[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) qv[j] = q[(size_t)h * D + lane * 8 + j] * 0.0625f; // rsqrt(256)
    float m = -INFINITY, l = 0.f, acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int t = w; t < L; t += W) {
        const size_t row = ((size_t)t * n_kv + kv) * D + lane * 8;
        float s = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) s = fmaf(qv[j], ld_kv(kc, row + j), s);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        const float m2 = fmaxf(m, s), c = __expf(m - m2), p = __expf(s - m2);
        l = l * c + p;
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = fmaf(p, ld_kv(vc, row + j), acc[j] * c);
        m = m2;
    }
    if (lane == 0) { s_m[w] = m; s_l[w] = l; }
#pragma unroll
    for (int j = 0; j < 8; ++j) s_acc[w][lane * 8 + j] = acc[j];
    __syncthreads();
    float mm = -INFINITY;
    for (int i = 0; i < W; ++i) mm = fmaxf(mm, s_m[i]);
    float ll = 0.f, o = 0.f;
    for (int i = 0; i < W; ++i) {
        const float c = s_m[i] == -INFINITY ? 0.f : __expf(s_m[i] - mm);
        ll += s_l[i] * c;
        o += s_acc[i][threadIdx.x] * c;
    }
    out[(size_t)h * D + threadIdx.x] = ll > 0.f ? o / ll : 0.f;
}

extern "C" __global__ void __launch_bounds__(256) attention_score(const float* q, const float* k_cache, const float* v_cache, float* output,
                                                                  uint32_t d_head, uint32_t seq_len, uint32_t current_pos,
                                                                  uint32_t n_kv_heads, uint32_t n_q_heads) {
    if (d_head != 256) return;
    attention_core<float>(q, k_cache, v_cache, output, (int)min(seq_len, current_pos), (int)n_kv_heads, (int)n_q_heads);
}
extern "C" __global__ void __launch_bounds__(256) attention_score_bf16(const float* q, const __nv_bfloat16* k_cache, const __nv_bfloat16* v_cache,
                                                                       float* output, uint32_t d_head, uint32_t seq_len, uint32_t current_pos,
                                                                       uint32_t n_kv_heads, uint32_t n_q_heads) {
    if (d_head != 256) return;
    attention_core<__nv_bfloat16>(q, k_cache, v_cache, output, (int)min(seq_len, current_pos), (int)n_kv_heads, (int)n_q_heads);
}
extern "C" __global__ void __launch_bounds__(256) attention_score_launcher(const float* q, const float* k_cache, const float* v_cache, float* output,
                                                                           uint32_t seq_len, uint32_t head_dim, uint32_t num_heads) {
    if (head_dim != 256) return;
    attention_core<float>(q, k_cache, v_cache, output, (int)seq_len, 4, (int)num_heads);
}
