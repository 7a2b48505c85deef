// Small kernels of the decode step: embedding gather, greedy argmax,
// stand-alone RMSNorm, and the L2 flush used by the timing harness.
#include "common.cuh"
#include "params.h"

// x = float(E[token]) : inference/embed.ls:16-24 with a bf16 table.  The token
// id is read from device memory so a captured graph can be replayed with a new
// token each step.
extern "C" __global__ void embed_bf16(const uint16_t* __restrict__ table, const int* __restrict__ token,
                                      float* __restrict__ out, int D) {
    pdl_wait();
    const size_t base = (size_t)token[0] * D;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < D; i += gridDim.x * blockDim.x)
        out[i] = bf16_bits_to_f32(table[base + i]);
}

// Greedy sampling: index of the maximum, FIRST maximum on ties (strict > in
// inference/reduce.ls:225-227 and src/launcher.s:1060-1063).  One CTA; the
// (value, index) pairs are combined with "greater value, else smaller index",
// which is order-independent, so the answer does not depend on the schedule.
// Also writes the winner into next_token (the next step's embed input) and
// advances *pos when given.
// cand_idx == NULL: x is the full vector and the index is the position; otherwise x[i] / cand_idx[i]
// are per-CTA candidates (value, row) left by the LM-head kernel.
extern "C" __global__ void __launch_bounds__(1024) argmax_f32(const float* __restrict__ x, int n, int* __restrict__ out_idx,
                                                              int* __restrict__ next_token, int* __restrict__ pos,
                                                              const int* __restrict__ cand_idx) {
    __shared__ float sv[32];
    __shared__ int si[32];
    pdl_wait();
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const float v = x[i];
        const int id = cand_idx ? cand_idx[i] : i;
        if (v > bv || (v == bv && id < bi)) { bv = v; bi = id; }
    }
    auto better = [](float v, int i, float bv2, int bi2) { return v > bv2 || (v == bv2 && i < bi2); };
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
    }
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    if (lane == 0) { sv[w] = bv; si[w] = bi; }
    __syncthreads();
    if (w == 0) {
        const int nw = blockDim.x >> 5;
        bv = lane < nw ? sv[lane] : -INFINITY;
        bi = lane < nw ? si[lane] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
        }
        if (lane == 0) {
            if (bi == 0x7fffffff) bi = 0; // all -inf / NaN: the reference's loop would keep index 0
            out_idx[0] = bi;
            if (next_token) next_token[0] = bi;
            if (pos) pos[0] += 1;
        }
    }
}

// Temperature + top-k sampling (the reference's `sample` kernel is described as "top-k sampling via parallel argmax
// reduction with temperature scaling", kernels/README.md:104-117; its shipped code only scales and takes the arg-max).
// One CTA.  The k largest logits are found by k block-wide arg-max passes in the order (larger value, then smaller
// index), each pass looking only at what comes after the previous winner in that order, so ties are resolved the same
// way every time; then p_i = exp((l_i - l_0) / T) / sum over the k, and the token is the first i whose cumulative
// probability exceeds u.  u comes from the same counter-based generator as the synthetic tensors: element `counter`
// (the decode position when pos != 0) of stream 7777 of `seed`, so a run can be repeated.  top_k is clamped to
// [1, 64]; temperature <= 0 means greedy.  Also writes next_token / advances *pos like argmax_f32.
__device__ __forceinline__ unsigned long long sm_mix64(unsigned long long z) {
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
extern "C" __global__ void __launch_bounds__(1024) topk_sample_f32(const float* __restrict__ x, int n, int* __restrict__ out_idx,
                                                                   int* __restrict__ next_token, int* __restrict__ pos, float temperature,
                                                                   int top_k, unsigned long long seed, unsigned long long counter,
                                                                   float* __restrict__ probs_out, int* __restrict__ idx_out) {
    __shared__ float sv[32];
    __shared__ int si[32];
    __shared__ float top_v[64];
    __shared__ int top_i[64];
    pdl_wait();
    const int k = temperature > 0.f ? min(max(top_k, 1), 64) : 1;
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = blockDim.x >> 5;
    auto better = [](float v, int i, float bv, int bi) { return v > bv || (v == bv && i < bi); };
    float last_v = INFINITY;
    int last_i = -1;
    for (int r = 0; r < k; ++r) {
        float bv = -INFINITY;
        int bi = 0x7fffffff;
        for (int i = threadIdx.x; i < n; i += blockDim.x) {
            const float v = x[i];
            const bool after = v < last_v || (v == last_v && i > last_i); // not taken yet
            if (after && better(v, i, bv, bi)) { bv = v; bi = i; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
        }
        if (lane == 0) { sv[w] = bv; si[w] = bi; }
        __syncthreads();
        if (w == 0) {
            bv = lane < nw ? sv[lane] : -INFINITY;
            bi = lane < nw ? si[lane] : 0x7fffffff;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
                const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
                if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
            }
            if (lane == 0) { top_v[r] = bv; top_i[r] = bi; }
        }
        __syncthreads();
        last_v = top_v[r];
        last_i = top_i[r];
    }
    if (threadIdx.x == 0) {
        int kk = k;
        while (kk > 1 && top_i[kk - 1] == 0x7fffffff) --kk; // fewer than k finite candidates
        int pick = 0;
        if (kk > 1) {
            const float inv_t = 1.0f / temperature;
            float p[64], sum = 0.f;
            for (int i = 0; i < kk; ++i) { p[i] = expf((top_v[i] - top_v[0]) * inv_t); sum += p[i]; }
            const unsigned long long c = pos ? (unsigned long long)pos[0] : counter;
            const unsigned long long h = sm_mix64(seed + 0x9E3779B97F4A7C15ull * (sm_mix64(7777ull ^ 0xD1342543DE82EF95ull) | 1ull));
            const unsigned bits = (unsigned)(sm_mix64(h + 0x9E3779B97F4A7C15ull * (c + 1)) >> 32);
            const float u = ((float)(bits >> 8) + 0.5f) * (1.0f / 16777216.0f);
            float acc = 0.f;
            bool found = false;
            pick = kk - 1; // rounding may leave the total a hair below u: the last candidate takes the rest
            for (int i = 0; i < kk; ++i) {
                const float pi = p[i] / sum;
                if (probs_out) probs_out[i] = pi;
                acc += pi;
                if (!found && u < acc) { pick = i; found = true; }
            }
        } else if (probs_out) probs_out[0] = 1.0f;
        if (idx_out) for (int i = 0; i < kk; ++i) idx_out[i] = top_i[i];
        int tok = top_i[pick];
        if (tok == 0x7fffffff) tok = 0;
        out_idx[0] = tok;
        if (next_token) next_token[0] = tok;
        if (pos) pos[0] += 1;
    }
}

// y = (x [+ r]) * w' * rsqrt(mean((x+r)^2) + eps), w' = 1+w or w (bf16 weight);
// inference/reduce.ls:21-147.  One CTA per row of D values.  sum_out (may be
// NULL) receives x+r.
extern "C" __global__ void __launch_bounds__(256) rmsnorm_f32(const float* __restrict__ x, const float* __restrict__ res,
                                                              const uint16_t* __restrict__ w, float* __restrict__ y,
                                                              float* __restrict__ sum_out, int D, float eps,
                                                              int one_plus_w) {
    __shared__ float red[40];
    pdl_wait();
    const size_t row = (size_t)blockIdx.x * D;
    float ss = 0.f;
    for (int i = threadIdx.x; i < D; i += blockDim.x) {
        const float v = x[row + i] + (res ? res[row + i] : 0.f);
        ss += v * v;
    }
    ss = block_sum(ss, red);
    const float rinv = rsqrtf(ss / (float)D + eps);
    for (int i = threadIdx.x; i < D; i += blockDim.x) {
        const float v = x[row + i] + (res ? res[row + i] : 0.f);
        if (sum_out) sum_out[row + i] = v;
        const float ww = bf16_bits_to_f32(w[i]);
        y[row + i] = v * rinv * (one_plus_w ? 1.0f + ww : ww);
    }
}

// Overwrites a buffer larger than L2 so the next timed kernel starts cold.
extern "C" __global__ void l2_flush(uint4* __restrict__ buf, size_t n16, uint32_t tag) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += (size_t)gridDim.x * blockDim.x)
        buf[i] = make_uint4(tag, tag, tag, tag);
}
