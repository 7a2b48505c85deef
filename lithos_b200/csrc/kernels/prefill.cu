// Prompt pass (prefill): the small kernels between the batched int4 projections (gemm_int4_*) when a chunk of up to 128
// prompt tokens goes through a layer at once.  The reference's prefill path is its dequantising GEMM
// (kernels/projection_gemm.sass:390-631) around the same element-wise / recurrence kernels as decoding
// (compiler/megakernel-link.ls:281-525 layer order); here every kernel takes a chunk [T, ...] and leaves exactly the
// state a token-by-token decode of the same tokens leaves: DeltaNet state, convolution ring (slot = position & 3), KV rows.
// All activations are fp32 except the projection inputs, which are rounded to fp16 (the decode step's contract).
#include "common.cuh"
#include "params.h"

// X[t, :] = float(E[token[t], :])                                   grid T, block 256
extern "C" __global__ void pf_embed(const uint16_t* __restrict__ table, const int* __restrict__ tokens, float* __restrict__ X, int D) {
    pdl_wait(); // launched with programmatic stream serialization: nothing of the previous kernel is read before this
    const size_t src = (size_t)tokens[blockIdx.x] * D, dst = (size_t)blockIdx.x * D;
    for (int i = threadIdx.x; i < D; i += blockDim.x) X[dst + i] = bf16_bits_to_f32(table[src + i]);
}

// [x[t, :] += add[t, :] when add is given;]  y16[t, :] = fp16( x[t, :] * rsqrt(mean x^2 + eps) * (1 + w) )
// grid T, block 256, D a multiple of 4                                                 (inference/reduce.ls:21-147)
extern "C" __global__ void __launch_bounds__(256) pf_rmsnorm_f16(float* __restrict__ X, const float* __restrict__ add,
                                                                 const uint16_t* __restrict__ w, __half* __restrict__ Y, int D, float eps) {
    pdl_wait(); // launched with programmatic stream serialization: nothing of the previous kernel is read before this
    __shared__ float red[33];
    float4* x4 = reinterpret_cast<float4*>(X + (size_t)blockIdx.x * D);
    const float4* a4 = add ? reinterpret_cast<const float4*>(add + (size_t)blockIdx.x * D) : nullptr;
    float ss = 0.f;
    for (int i = threadIdx.x; i < D / 4; i += 256) {
        float4 v = x4[i];
        if (a4) {
            const float4 a = a4[i];
            v.x += a.x; v.y += a.y; v.z += a.z; v.w += a.w;
            x4[i] = v;
        }
        ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
    ss = block_sum(ss, red);
    const float rinv = rsqrtf(ss / (float)D + eps);
    for (int i = threadIdx.x; i < D / 4; i += 256) { // the thread re-reads what it wrote itself
        const float4 v = x4[i];
        const uint2 ww = *reinterpret_cast<const uint2*>(w + 4 * i);
        const __half2 lo = __floats2half2_rn(v.x * rinv * (1.0f + __uint_as_float(ww.x << 16)), v.y * rinv * (1.0f + __uint_as_float(ww.x & 0xffff0000u)));
        const __half2 hi = __floats2half2_rn(v.z * rinv * (1.0f + __uint_as_float(ww.y << 16)), v.w * rinv * (1.0f + __uint_as_float(ww.y & 0xffff0000u)));
        uint2 o;
        o.x = *reinterpret_cast<const uint32_t*>(&lo);
        o.y = *reinterpret_cast<const uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(Y + (size_t)blockIdx.x * D + 4 * i) = o;
    }
}

// The DeltaNet front end of a chunk: causal 4-tap convolution over time, SiLU, per-head L2 norm of q and k, q / sqrt(128).
// One block per (token, head of q, k or v): grid (T, 2*HK + HV), thread = channel.  The three earlier tokens of a channel are
// rows of the same projection buffer, or, before the chunk's first token, slots of the ring history (slot = position & 3),
// which this kernel only reads: pf_dn_ring records the chunk's last positions afterwards.
// proj [T, ld]: q | k | v | z columns of the fused projection.  Writes q, k [T, HK, 128], v [T, HV, 128] (fp32).
//                                                                        (inference/recur.ls:12-40, reduce.ls:153-207)
extern "C" __global__ void __launch_bounds__(128) pf_dn_frontend(const float* __restrict__ proj, int ld, const uint16_t* __restrict__ conv_w,
                                                                 const float* __restrict__ ring, float* __restrict__ q, float* __restrict__ k,
                                                                 float* __restrict__ v, int HK, int HV, int pos0, int T) {
    pdl_wait(); // launched with programmatic stream serialization: nothing of the previous kernel is read before this
    __shared__ float red[4];
    const int QK = HK * 128, C = 2 * QK + HV * 128;
    const int s = blockIdx.x, b = blockIdx.y, t = threadIdx.x;
    const int kind = b < HK ? 0 : b < 2 * HK ? 1 : 2, head = kind == 0 ? b : kind == 1 ? b - HK : b - 2 * HK;
    const int c = (kind == 0 ? 0 : kind == 1 ? QK : 2 * QK) + head * 128 + t;
    auto past = [&](int back) { // the channel's raw value `back` tokens ago
        return s >= back ? proj[(size_t)(s - back) * ld + c] : ring[(size_t)((pos0 + s - back) & 3) * C + c];
    };
    float y = bf16_bits_to_f32(conv_w[c]) * proj[(size_t)s * ld + c];
    y = fmaf(bf16_bits_to_f32(conv_w[C + c]), past(1), y);
    y = fmaf(bf16_bits_to_f32(conv_w[2 * C + c]), past(2), y);
    y = fmaf(bf16_bits_to_f32(conv_w[3 * C + c]), past(3), y);
    y = siluf_dev(y);
    if (kind == 2) { v[((size_t)s * HV + head) * 128 + t] = y; return; }
    float n2 = warp_sum(y * y);
    if ((t & 31) == 0) red[t >> 5] = n2;
    __syncthreads();
    n2 = (red[0] + red[1]) + (red[2] + red[3]);
    if (kind == 0) q[((size_t)s * HK + head) * 128 + t] = y * rsqrtf(n2) * 0.08838834764831845f;
    else k[((size_t)s * HK + head) * 128 + t] = y * rsqrtf(n2);
}

// ring[(pos0 + s) & 3][c] = proj[s][c] for the chunk's last (up to four) tokens: the history the next chunk, or the decode
// step, continues from.  grid ceil(C / 256), block 256
extern "C" __global__ void pf_dn_ring(const float* __restrict__ proj, int ld, float* __restrict__ ring, int C, int pos0, int T) {
    pdl_wait(); // launched with programmatic stream serialization: nothing of the previous kernel is read before this
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    for (int s = T > 4 ? T - 4 : 0; s < T; ++s) ring[(size_t)((pos0 + s) & 3) * C + c] = proj[(size_t)s * ld + c];
}

// decay and beta of a chunk: a = in_proj_a . xn, b = in_proj_b . xn per value head, then
// g = exp(-exp(A_log) softplus(a + dt_bias)), beta = sigmoid(b).  A block owns one head and 8 consecutive tokens (the two
// weight rows are read once per 8 tokens); its four warps take a quarter of the hidden dimension each and the quarters are
// added in warp order.  grid (ceil(T/8), HV), block 128; H a multiple of 8.
extern "C" __global__ void __launch_bounds__(128) pf_ab_gate(const __half* __restrict__ xn, const uint16_t* __restrict__ proj_a,
                                                             const uint16_t* __restrict__ proj_b, const float* __restrict__ a_log,
                                                             const uint16_t* __restrict__ dt_bias, float* __restrict__ g,
                                                             float* __restrict__ beta, int HV, int H, int T) {
    pdl_wait(); // launched with programmatic stream serialization: nothing of the previous kernel is read before this
    __shared__ float red[4][16];
    const int s0 = blockIdx.x * 8, h = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint4* ra = reinterpret_cast<const uint4*>(proj_a + (size_t)h * H);
    const uint4* rb = reinterpret_cast<const uint4*>(proj_b + (size_t)h * H);
    float a[8], b[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) a[j] = b[j] = 0.f;
    const int n8 = H / 8, per = (n8 + 3) / 4;
    for (int i = warp * per + lane; i < min(n8, (warp + 1) * per); i += 32) {
        const uint4 wa = __ldg(ra + i), wb = __ldg(rb + i);
        const uint32_t aw[4] = {wa.x, wa.y, wa.z, wa.w}, bw[4] = {wb.x, wb.y, wb.z, wb.w};
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int s = min(s0 + j, T - 1); // tokens past the chunk repeat the last one; they are not stored
            const uint4 xx = *(reinterpret_cast<const uint4*>(xn + (size_t)s * H) + i);
            const uint32_t xw[4] = {xx.x, xx.y, xx.z, xx.w};
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const float2 xf = __half22float2(*reinterpret_cast<const __half2*>(&xw[q]));
                a[j] = fmaf(__uint_as_float(aw[q] << 16), xf.x, a[j]);
                a[j] = fmaf(__uint_as_float(aw[q] & 0xffff0000u), xf.y, a[j]);
                b[j] = fmaf(__uint_as_float(bw[q] << 16), xf.x, b[j]);
                b[j] = fmaf(__uint_as_float(bw[q] & 0xffff0000u), xf.y, b[j]);
            }
        }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        a[j] = warp_sum(a[j]);
        b[j] = warp_sum(b[j]);
        if (lane == 0) {
            red[warp][j] = a[j];
            red[warp][8 + j] = b[j];
        }
    }
    __syncthreads();
    const int j = threadIdx.x;
    if (j < 8 && s0 + j < T) {
        const float av = (red[0][j] + red[1][j]) + (red[2][j] + red[3][j]);
        const float bv = (red[0][8 + j] + red[1][8 + j]) + (red[2][8 + j] + red[3][8 + j]);
        const float tt = av + bf16_bits_to_f32(dt_bias[h]);
        const float sp = tt > 20.f ? tt : log1pf(expf(tt));
        g[(size_t)(s0 + j) * HV + h] = expf(-expf(a_log[h]) * sp);
        beta[(size_t)(s0 + j) * HV + h] = 1.0f / (1.0f + expf(-bv));
    }
}

// y16[t, h, :] = fp16( o * rsqrt(mean_head o^2 + eps) * w * silu(z) ): the out projection's input.  One warp per (token, head).
// o [T, HV, 128]; z = proj + z_off with row stride ld.            grid (T, ceil(HV/4)), block 128
extern "C" __global__ void __launch_bounds__(128) pf_headnorm_gate_f16(const float* __restrict__ o, const float* __restrict__ proj, int ld,
                                                                       int z_off, const float* __restrict__ w, __half* __restrict__ y,
                                                                       int HV, float eps) {
    pdl_wait(); // launched with programmatic stream serialization: nothing of the previous kernel is read before this
    const int s = blockIdx.x, h = blockIdx.y * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (h >= HV) return;
    const float4 v = *reinterpret_cast<const float4*>(o + ((size_t)s * HV + h) * 128 + lane * 4);
    const float4 z = *reinterpret_cast<const float4*>(proj + (size_t)s * ld + z_off + h * 128 + lane * 4);
    const float4 ww = *reinterpret_cast<const float4*>(w + lane * 4);
    const float r = rsqrtf(warp_sum(v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w) * (1.0f / 128.0f) + eps);
    __half* dst = y + ((size_t)s * HV + h) * 128 + lane * 4;
    dst[0] = __float2half_rn(v.x * r * ww.x * siluf_dev(z.x));
    dst[1] = __float2half_rn(v.y * r * ww.y * siluf_dev(z.y));
    dst[2] = __float2half_rn(v.z * r * ww.z * siluf_dev(z.z));
    dst[3] = __float2half_rn(v.w * r * ww.w * siluf_dev(z.w));
}

// SwiGLU of a chunk: gu [T, 2I] in interleaved 64-wide (gate, up) blocks -> y16 [T, I] = silu(gate) * up    (kernels.ls:61-66)
// four outputs per thread; total4 = T * I / 4 (fits 32 bits: a chunk has at most 256 tokens)
extern "C" __global__ void pf_swiglu_f16(const float* __restrict__ gu, __half* __restrict__ y, int I, int total4) {
    pdl_wait(); // launched with programmatic stream serialization: nothing of the previous kernel is read before this
    const int I4 = I / 4;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total4; i += gridDim.x * blockDim.x) {
        const int s = i / I4, n = (i - s * I4) * 4, blk = n >> 6, j = n & 63;
        const float* row = gu + (size_t)s * 2 * I + (size_t)blk * 128;
        const float4 gt = *reinterpret_cast<const float4*>(row + j), up = *reinterpret_cast<const float4*>(row + 64 + j);
        const __half2 lo = __floats2half2_rn(siluf_dev(gt.x) * up.x, siluf_dev(gt.y) * up.y);
        const __half2 hi = __floats2half2_rn(siluf_dev(gt.z) * up.z, siluf_dev(gt.w) * up.w);
        uint2 o;
        o.x = *reinterpret_cast<const uint32_t*>(&lo);
        o.y = *reinterpret_cast<const uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(y + (size_t)i * 4) = o;
    }
}

// x += y, four values per thread (n4 = n / 4)
extern "C" __global__ void pf_add(float4* __restrict__ x, const float4* __restrict__ y, int n4) {
    pdl_wait(); // launched with programmatic stream serialization: nothing of the previous kernel is read before this
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += gridDim.x * blockDim.x) {
        float4 a = x[i];
        const float4 b = y[i];
        a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
        x[i] = a;
    }
}

// ---- causal attention of a chunk ---------------------------------------------------------------------------------
// The decode step runs q/k norm, RoPE, the KV append and the attention of ONE token in one kernel (attention_mma.cu;
// inference/attend.ls:85-191, attend_full.ls:186-248).  For a chunk of T prompt tokens the same work is two kernels:
// pf_attn_prepare does the per-token part with the decode kernel's own routine (same bits in the cache rows and the
// same queries), pf_attn_chunk then attends all T tokens at once, token s over the cache rows [0, pos0 + s].
#include "attention_core.cuh"

// grid T, block 256: token s of the chunk.  Queries -> (qh, ql) as two bf16 terms, pre-scaled by log2(e)/sqrt(256);
// key -> norm, RoPE, bf16 -> cache row pos0+s; value -> bf16 -> cache row pos0+s.
extern "C" __global__ void __launch_bounds__(256) pf_attn_prepare(const __grid_constant__ lb_pf_attn_params p) {
    pdl_wait();
    __shared__ float cs_s[128], sn_s[128];
    __shared__ __align__(16) float row_s[8][AT_D];
    const int s = blockIdx.x, t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const int pos = p.pos0 + s;
    if (t < p.rot_dims / 2) { // the decode kernel's angle reduction: product and reduction modulo 2 pi in double
        const double a = (double)pos * p.rope_freq[t];
        const double k = rint(a * 0.15915494309189535);
        const float r = (float)fma(-k, 6.283185307179586, a);
        sincosf(r, &sn_s[t], &cs_s[t]);
    }
    __syncthreads();
    const float qscale = rsqrtf((float)AT_D) * 1.4426950408889634f; // scores in log2 units
    const float* row = p.proj + (size_t)s * p.ld;
    const size_t nq = (size_t)2 * p.HQ * AT_D, nkv = (size_t)p.HKV * AT_D;
    for (int r = warp; r < p.HQ + p.HKV; r += 8) {
        float* dst = row_s[warp];
        if (r < p.HQ) {
            warp_norm_rope(row, (size_t)r * 512, 1, p.q_norm_w, dst, cs_s, sn_s, p.rot_dims, p.eps, qscale);
            __syncwarp();
            const size_t o = ((size_t)s * p.HQ + r) * AT_D + lane * 8;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float q = dst[lane * 8 + j];
                const __nv_bfloat16 h = __float2bfloat16_rn(q);
                reinterpret_cast<__nv_bfloat16*>(p.qh)[o + j] = h;
                reinterpret_cast<__nv_bfloat16*>(p.ql)[o + j] = __float2bfloat16_rn(q - __bfloat162float(h));
            }
        } else {
            const int kv = r - p.HQ;
            warp_norm_rope(row + nq, (size_t)kv * AT_D, 1, p.k_norm_w, dst, cs_s, sn_s, p.rot_dims, p.eps, 1.0f);
            __syncwarp();
            const size_t o = ((size_t)pos * p.HKV + kv) * AT_D + lane * 8;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                reinterpret_cast<__nv_bfloat16*>(p.k_cache)[o + j] = __float2bfloat16_rn(dst[lane * 8 + j]);
                reinterpret_cast<__nv_bfloat16*>(p.v_cache)[o + j] = __float2bfloat16_rn(row[nq + nkv + (size_t)kv * AT_D + lane * 8 + j]);
            }
        }
        __syncwarp();
    }
}

#define PA_ROWS LB_PF_ATTN_ROWS   // query rows per CTA
#define PA_WARPS (PA_ROWS / 16)  // warps per CTA, 16 query rows each
#define PA_KV 32                 // cache rows per staged block
#define PA_STRIDE 528            // bytes per staged row: 512 + 16 (8 rows on 8 different bank groups)
#define PA_THREADS LB_PF_ATTN_THREADS
// dynamic shared memory: qh | ql [PA_ROWS][528], then two stages of K | V [PA_KV][528]
static_assert(PA_THREADS == 32 * PA_WARPS && LB_PF_ATTN_SMEM == 2 * PA_ROWS * PA_STRIDE + 2 * 2 * PA_KV * PA_STRIDE, "launch geometry");

__device__ __forceinline__ void pa_mma(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void pa_ldsm(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void pa_ldsm_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void pa_cp16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void pa_split(float x, float y, uint32_t& hi, uint32_t& lo) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(x, y);
    const float2 hf = __bfloat1622float2(h);
    const __nv_bfloat162 l = __floats2bfloat162_rn(x - hf.x, y - hf.y);
    hi = *reinterpret_cast<const uint32_t*>(&h);
    lo = *reinterpret_cast<const uint32_t*>(&l);
}

// grid (ceil(T*G / PA_ROWS), HKV), block PA_THREADS.  Query row R of a KV head = (token R / G, head R % G): a warp's 16 rows
// are 16/G consecutive tokens, so their causal limits differ by a few rows only.  S = Q K^T and O = P V as
// mma.sync.m16n8k16 bf16 with Q and P split into two bf16 terms (the decode kernel's precision: 16 bits of Q and P, K and V
// exact in bf16), online soft-max per row in the four lanes that hold the row, cache rows staged 32 at a time by cp.async
// in two stages shared by the CTA's warps.  The M side is query rows x heads here, which is why this is not the decode
// kernel with a loop around it: a cache row is read once per CTA instead of once per token.
extern "C" __global__ void __launch_bounds__(PA_THREADS) pf_attn_chunk(const __grid_constant__ lb_pf_attn_params p) {
    extern __shared__ __align__(16) unsigned char pa_sm[];
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const int fg = lane >> 2, ft = lane & 3;
    const int kv = blockIdx.y, G = p.HQ / p.HKV;
    const int R0 = blockIdx.x * PA_ROWS;
    const int n_rows = p.T * G;
    unsigned char* qh_s = pa_sm;
    unsigned char* ql_s = qh_s + PA_ROWS * PA_STRIDE;
    unsigned char* kv_s = ql_s + PA_ROWS * PA_STRIDE; // stage st: K at st * 2 * PA_KV * PA_STRIDE, V after it
    pdl_wait();

    // the CTA's query rows (rows past the chunk repeat the last one; they are never stored)
    for (int i = t; i < PA_ROWS * 32; i += PA_THREADS) {
        const int r = i >> 5, c = i & 31;
        const int R = min(R0 + r, n_rows - 1), s = R / G, g = R - s * G;
        const size_t src = (((size_t)s * p.HQ + kv * G + g) * AT_D) * 2 + c * 16;
        pa_cp16(smem_u32(qh_s + r * PA_STRIDE + c * 16), reinterpret_cast<const unsigned char*>(p.qh) + src);
        pa_cp16(smem_u32(ql_s + r * PA_STRIDE + c * 16), reinterpret_cast<const unsigned char*>(p.ql) + src);
    }
    // last cache row any row of this CTA may see, and of this warp
    const int s_cta = min(R0 + PA_ROWS - 1, n_rows - 1) / G;
    const int last_row = p.pos0 + s_cta;
    const int n_blocks = last_row / PA_KV + 1;
    const size_t row_bytes = (size_t)p.HKV * AT_D * 2;
    auto stage = [&](int b) { // rows past the last one repeat it (finite values; masked below)
        unsigned char* dst = kv_s + (b & 1) * (2 * PA_KV * PA_STRIDE);
        for (int i = t; i < 2 * PA_KV * 32; i += PA_THREADS) {
            const int which = i / (PA_KV * 32), r = (i >> 5) % PA_KV, c = i & 31;
            const int row = min(b * PA_KV + r, last_row);
            const unsigned char* base = reinterpret_cast<const unsigned char*>(which ? p.v_cache : p.k_cache);
            pa_cp16(smem_u32(dst + (which * PA_KV + r) * PA_STRIDE + c * 16), base + (size_t)row * row_bytes + (size_t)kv * AT_D * 2 + c * 16);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    stage(0);

    // rows fg and fg+8 of the warp's tile
    int lim[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) lim[i] = p.pos0 + min(R0 + warp * 16 + fg + 8 * i, n_rows - 1) / G;
    const int warp_last = p.pos0 + min(R0 + warp * 16 + 15, n_rows - 1) / G;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    float acc[32][4];
#pragma unroll
    for (int nb = 0; nb < 32; ++nb) acc[nb][0] = acc[nb][1] = acc[nb][2] = acc[nb][3] = 0.f;
    // ldmatrix lane addresses.  A (Q rows, x4): (rows 0-7, dims c..c+7), (rows 8-15, c), (rows 0-7, c+8), (rows 8-15, c+8)
    const uint32_t a_off = (warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * PA_STRIDE + (lane >> 4) * 16;
    const uint32_t qh_lane = smem_u32(qh_s) + a_off, ql_lane = smem_u32(ql_s) + a_off;
    // K (x4): (rows 0-7, dims c..c+7), (rows 0-7, c+8), (rows 8-15, c), (rows 8-15, c+8)
    const uint32_t k_off = ((lane & 7) + ((lane >> 4) << 3)) * PA_STRIDE + ((lane >> 3) & 1) * 16;
    // V (x4, transposed): (rows 0-7, dims d..d+7), (rows 8-15, d), (rows 0-7, d+8), (rows 8-15, d+8)
    const uint32_t v_off = ((lane & 7) + ((lane >> 3) & 1) * 8) * PA_STRIDE + (lane >> 4) * 16;

    for (int b = 0; b < n_blocks; ++b) {
        if (b + 1 < n_blocks) {
            stage(b + 1);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();
        if (b * PA_KV <= warp_last) {
            const uint32_t k_addr = smem_u32(kv_s + (b & 1) * (2 * PA_KV * PA_STRIDE)), v_addr = k_addr + PA_KV * PA_STRIDE;
            float sc[4][4];
#pragma unroll
            for (int j = 0; j < 4; ++j) sc[j][0] = sc[j][1] = sc[j][2] = sc[j][3] = 0.f;
#pragma unroll
            for (int c = 0; c < 16; ++c) {
                uint32_t h0, h1, h2, h3, l0, l1, l2, l3;
                pa_ldsm(qh_lane + c * 32, h0, h1, h2, h3);
                pa_ldsm(ql_lane + c * 32, l0, l1, l2, l3);
#pragma unroll
                for (int jj = 0; jj < 2; ++jj) {
                    uint32_t b00, b01, b10, b11;
                    pa_ldsm(k_addr + k_off + jj * 16 * PA_STRIDE + c * 32, b00, b01, b10, b11);
                    pa_mma(sc[2 * jj], h0, h1, h2, h3, b00, b01);
                    pa_mma(sc[2 * jj], l0, l1, l2, l3, b00, b01);
                    pa_mma(sc[2 * jj + 1], h0, h1, h2, h3, b10, b11);
                    pa_mma(sc[2 * jj + 1], l0, l1, l2, l3, b10, b11);
                }
            }
            // sc[j][0..1]: row fg, cache rows b*32 + 8j + 2ft, +1; sc[j][2..3]: row fg+8
            float corr[2];
            uint32_t ph[4][2], pl[4][2]; // [j][row half]: the probabilities as bf16 pairs
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                float mx = -INFINITY;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int r0 = b * PA_KV + 8 * j + 2 * ft;
                    if (r0 > lim[i]) sc[j][2 * i] = -INFINITY;
                    if (r0 + 1 > lim[i]) sc[j][2 * i + 1] = -INFINITY;
                    mx = fmaxf(mx, fmaxf(sc[j][2 * i], sc[j][2 * i + 1]));
                }
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
                const float m_new = fmaxf(m_run[i], mx); // finite from block 0 on: cache row 0 is visible to every query row
                corr[i] = exp2f(m_run[i] - m_new);       // exp2f(-inf) = 0 on the first block
                float ps = 0.f;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float p0 = exp2f(sc[j][2 * i] - m_new), p1 = exp2f(sc[j][2 * i + 1] - m_new);
                    ps += p0 + p1;
                    pa_split(p0, p1, ph[j][i], pl[j][i]);
                }
                ps += __shfl_xor_sync(0xffffffffu, ps, 1);
                ps += __shfl_xor_sync(0xffffffffu, ps, 2);
                l_run[i] = fmaf(l_run[i], corr[i], ps);
                m_run[i] = m_new;
            }
            // O += P V: k-step kk = cache rows 16kk..16kk+15 (score blocks 2kk, 2kk+1), n-block nb = dims 8nb..8nb+7
#pragma unroll
            for (int nb = 0; nb < 32; nb += 2) {
                acc[nb][0] *= corr[0]; acc[nb][1] *= corr[0]; acc[nb][2] *= corr[1]; acc[nb][3] *= corr[1];
                acc[nb + 1][0] *= corr[0]; acc[nb + 1][1] *= corr[0]; acc[nb + 1][2] *= corr[1]; acc[nb + 1][3] *= corr[1];
#pragma unroll
                for (int kk = 0; kk < 2; ++kk) {
                    uint32_t v0, v1, v2, v3;
                    pa_ldsm_t(v_addr + v_off + kk * 16 * PA_STRIDE + nb * 16, v0, v1, v2, v3);
                    pa_mma(acc[nb], ph[2 * kk][0], ph[2 * kk][1], ph[2 * kk + 1][0], ph[2 * kk + 1][1], v0, v1);
                    pa_mma(acc[nb], pl[2 * kk][0], pl[2 * kk][1], pl[2 * kk + 1][0], pl[2 * kk + 1][1], v0, v1);
                    pa_mma(acc[nb + 1], ph[2 * kk][0], ph[2 * kk][1], ph[2 * kk + 1][0], ph[2 * kk + 1][1], v2, v3);
                    pa_mma(acc[nb + 1], pl[2 * kk][0], pl[2 * kk][1], pl[2 * kk + 1][0], pl[2 * kk + 1][1], v2, v3);
                }
            }
        }
        __syncthreads(); // every warp is done with this stage before block b+2 overwrites it
    }

    // out[s][hq][dim] = fp16( O / l * sigmoid(gate) ): lane (fg, ft) holds dims 8nb + 2ft, +1 of rows fg and fg+8
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int R = R0 + warp * 16 + fg + 8 * i;
        if (R >= n_rows) continue;
        const int s = R / G, hq = kv * G + (R - s * G);
        const float inv = 1.0f / l_run[i];
        const float* gate = p.proj + (size_t)s * p.ld + (size_t)hq * 512 + 256;
        __half2* dst = reinterpret_cast<__half2*>(p.out + ((size_t)s * p.HQ + hq) * AT_D);
#pragma unroll
        for (int nb = 0; nb < 32; ++nb) {
            const float2 gt = *reinterpret_cast<const float2*>(gate + 8 * nb + 2 * ft);
            dst[4 * nb + ft] = __floats2half2_rn(acc[nb][2 * i] * inv * sigmoidf_dev(gt.x), acc[nb][2 * i + 1] * inv * sigmoidf_dev(gt.y));
        }
    }
}
