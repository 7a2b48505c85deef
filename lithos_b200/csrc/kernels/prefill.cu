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

// y16[t, :] = fp16( x[t, :] * rsqrt(mean x^2 + eps) * (1 + w) )      grid T, block 256   (inference/reduce.ls:21-147)
extern "C" __global__ void __launch_bounds__(256) pf_rmsnorm_f16(const float* __restrict__ X, const uint16_t* __restrict__ w,
                                                                 __half* __restrict__ Y, int D, float eps) {
    pdl_wait(); // launched with programmatic stream serialization: nothing of the previous kernel is read before this
    __shared__ float red[33];
    const float* x = X + (size_t)blockIdx.x * D;
    float ss = 0.f;
    for (int i = threadIdx.x; i < D; i += blockDim.x) ss += x[i] * x[i];
    ss = block_sum(ss, red);
    const float rinv = rsqrtf(ss / (float)D + eps);
    for (int i = threadIdx.x; i < D; i += blockDim.x)
        Y[(size_t)blockIdx.x * D + i] = __float2half_rn(x[i] * rinv * (1.0f + bf16_bits_to_f32(w[i])));
}

// The DeltaNet front end of a chunk: causal 4-tap convolution over time (ring history), SiLU, per-head L2 norm of q and k,
// q / sqrt(128).  One block per head of q, k or v (blockIdx.x < 2*HK + HV), thread = channel, the chunk's tokens in order.
// proj [T, ld]: q | k | v | z columns of the fused projection.  Writes q, k [T, HK, 128], v [T, HV, 128] (fp32) and the ring
// slots of the chunk's last four positions.                            (inference/recur.ls:12-40, reduce.ls:153-207)
extern "C" __global__ void __launch_bounds__(128) pf_dn_frontend(const float* __restrict__ proj, int ld, const uint16_t* __restrict__ conv_w,
                                                                 float* __restrict__ ring, float* __restrict__ q, float* __restrict__ k,
                                                                 float* __restrict__ v, int HK, int HV, int pos0, int T) {
    pdl_wait(); // launched with programmatic stream serialization: nothing of the previous kernel is read before this
    __shared__ float red[4];
    const int QK = HK * 128, C = 2 * QK + HV * 128;
    const int b = blockIdx.x, t = threadIdx.x;
    const int kind = b < HK ? 0 : b < 2 * HK ? 1 : 2, head = kind == 0 ? b : kind == 1 ? b - HK : b - 2 * HK;
    const int c = (kind == 0 ? 0 : kind == 1 ? QK : 2 * QK) + head * 128 + t;
    const float w0 = bf16_bits_to_f32(conv_w[c]), w1 = bf16_bits_to_f32(conv_w[C + c]), w2 = bf16_bits_to_f32(conv_w[2 * C + c]),
                w3 = bf16_bits_to_f32(conv_w[3 * C + c]);
    float h1 = ring[(size_t)((pos0 + 3) & 3) * C + c], h2 = ring[(size_t)((pos0 + 2) & 3) * C + c], h3 = ring[(size_t)((pos0 + 1) & 3) * C + c];
    for (int s = 0; s < T; ++s) {
        const float x = proj[(size_t)s * ld + c];
        float y = w0 * x;
        y = fmaf(w1, h1, y);
        y = fmaf(w2, h2, y);
        y = fmaf(w3, h3, y);
        y = siluf_dev(y);
        h3 = h2; h2 = h1; h1 = x;
        if (s >= T - 4) ring[(size_t)((pos0 + s) & 3) * C + c] = x;
        if (kind == 2) { v[((size_t)s * HV + head) * 128 + t] = y; continue; }
        float n2 = warp_sum(y * y);
        __syncthreads();
        if ((t & 31) == 0) red[t >> 5] = n2;
        __syncthreads();
        n2 = (red[0] + red[1]) + (red[2] + red[3]);
        if (kind == 0) q[((size_t)s * HK + head) * 128 + t] = y * rsqrtf(n2) * 0.08838834764831845f;
        else k[((size_t)s * HK + head) * 128 + t] = y * rsqrtf(n2);
    }
}

// decay and beta of a chunk: a = in_proj_a . xn, b = in_proj_b . xn per value head, then
// g = exp(-exp(A_log) softplus(a + dt_bias)), beta = sigmoid(b).  One warp per (token, head): grid (T, ceil(HV/4)), block 128.
extern "C" __global__ void __launch_bounds__(128) pf_ab_gate(const __half* __restrict__ xn, const uint16_t* __restrict__ proj_a,
                                                             const uint16_t* __restrict__ proj_b, const float* __restrict__ a_log,
                                                             const uint16_t* __restrict__ dt_bias, float* __restrict__ g,
                                                             float* __restrict__ beta, int HV, int H) {
    pdl_wait(); // launched with programmatic stream serialization: nothing of the previous kernel is read before this
    const int s = blockIdx.x, h = blockIdx.y * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (h >= HV) return;
    const __half* x = xn + (size_t)s * H;
    const uint16_t *ra = proj_a + (size_t)h * H, *rb = proj_b + (size_t)h * H;
    float a = 0.f, b = 0.f;
    for (int i = lane; i < H; i += 32) {
        const float xv = __half2float(x[i]);
        a = fmaf(bf16_bits_to_f32(ra[i]), xv, a);
        b = fmaf(bf16_bits_to_f32(rb[i]), xv, b);
    }
    a = warp_sum(a);
    b = warp_sum(b);
    if (lane == 0) {
        const float tt = a + bf16_bits_to_f32(dt_bias[h]);
        const float sp = tt > 20.f ? tt : log1pf(expf(tt));
        g[(size_t)s * HV + h] = expf(-expf(a_log[h]) * sp);
        beta[(size_t)s * HV + h] = 1.0f / (1.0f + expf(-b));
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
extern "C" __global__ void pf_swiglu_f16(const float* __restrict__ gu, __half* __restrict__ y, int I, long long total) {
    pdl_wait(); // launched with programmatic stream serialization: nothing of the previous kernel is read before this
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long s = i / I;
        const int n = (int)(i - s * I), blk = n >> 6, j = n & 63;
        const float* row = gu + s * 2 * I + (long long)blk * 128;
        y[i] = __float2half_rn(siluf_dev(row[j]) * row[64 + j]);
    }
}

extern "C" __global__ void pf_add(float* __restrict__ x, const float* __restrict__ y, long long n) {
    pdl_wait(); // launched with programmatic stream serialization: nothing of the previous kernel is read before this
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) x[i] += y[i];
}
extern "C" __global__ void pf_f32_to_f16(const float* __restrict__ x, __half* __restrict__ y, long long n) {
    pdl_wait(); // launched with programmatic stream serialization: nothing of the previous kernel is read before this
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) y[i] = __float2half_rn(x[i]);
}
