// The whole DeltaNet mixer of one layer for ONE (value head, 32-column slab) unit, run by a team of 128 threads:
// shared by the stand-alone kernel (deltanet.cu: one CTA per unit) and the persistent decode chain (chain.cu: four
// teams per CTA).  `sync` is the team's barrier; inputs produced earlier in the SAME launch (qkvz, xn) are read
// through L2 only (ld.global.cg).
#pragma once
#include "common.cuh"
#include "params.h"

#define DN_D 128
#define DN_COLS 32      // state columns per unit
#define DN_THREADS 128  // 8 column-quads x 16 row phases

struct __align__(16) dn_unit_smem {
    float part[16][DN_COLS];
    float ks[DN_D], qs[DN_D], vs[DN_COLS], red[16];
};

// sum over the team's 128 threads (4 warps, fixed order); every thread gets the total
template <class Sync>
__device__ __forceinline__ float dn_unit_sum(float v, float (&red)[16], int t, Sync sync) {
    v = warp_sum(v);
    sync(); // earlier readers of red are done
    if ((t & 31) == 0) red[t >> 5] = v;
    sync();
    return (red[0] + red[1]) + (red[2] + red[3]);
}

// four sums at once (each added in the same order as dn_unit_sum would): one exchange through shared memory instead of four
template <class Sync>
__device__ __forceinline__ void dn_unit_sum4(float& a, float& b, float& c, float& d, float (&red)[16], int t, Sync sync) {
    a = warp_sum(a); b = warp_sum(b); c = warp_sum(c); d = warp_sum(d);
    sync(); // earlier readers of red are done
    if ((t & 31) == 0) {
        const int w = t >> 5;
        red[w] = a; red[4 + w] = b; red[8 + w] = c; red[12 + w] = d;
    }
    sync();
    a = (red[0] + red[1]) + (red[2] + red[3]);
    b = (red[4] + red[5]) + (red[6] + red[7]);
    c = (red[8] + red[9]) + (red[10] + red[11]);
    d = (red[12] + red[13]) + (red[14] + red[15]);
}

// in_proj_a / in_proj_b of one value head: the partial dot products of thread t of a team with the normalised layer input
// (bf16 rows, fp16 input, fp32 accumulate; ROWS = 2: both rows, ROWS = 1: the row `row0`).  All loads are issued before the
// first use, so the dot products cost one trip to L2, not one per piece (hidden 5120 = exactly one pass of five
// 8-element pieces per thread).
template <int ROWS>
__device__ __forceinline__ void dn_gate_dot(const lb_dn_layer_params& p, const uint16_t* row0, const uint16_t* row1, int t, float& a, float& b) {
    const uint4* ra = reinterpret_cast<const uint4*>(row0);
    const uint4* rb = reinterpret_cast<const uint4*>(row1);
    const uint4* xv = reinterpret_cast<const uint4*>(p.xn);
    const int n8 = p.hidden / 8;
    a = b = 0.f;
    for (int base = 0; base < n8; base += 5 * DN_THREADS) {
        uint4 wa[5], wb[5], xx[5];
#pragma unroll
        for (int j = 0; j < 5; ++j) {
            const int i = base + j * DN_THREADS + t;
            const bool on = i < n8;
            wa[j] = on ? __ldg(ra + i) : make_uint4(0u, 0u, 0u, 0u);
            if (ROWS == 2) wb[j] = on ? __ldg(rb + i) : make_uint4(0u, 0u, 0u, 0u);
            xx[j] = on ? __ldcg(xv + i) : make_uint4(0u, 0u, 0u, 0u);
        }
#pragma unroll
        for (int j = 0; j < 5; ++j) {
            const uint32_t aw[4] = {wa[j].x, wa[j].y, wa[j].z, wa[j].w};
            const uint32_t xw[4] = {xx[j].x, xx[j].y, xx[j].z, xx[j].w};
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const float2 xf = __half22float2(*reinterpret_cast<const __half2*>(&xw[q]));
                a = fmaf(__uint_as_float(aw[q] << 16), xf.x, a);
                a = fmaf(__uint_as_float(aw[q] & 0xffff0000u), xf.y, a);
                if (ROWS == 2) {
                    const uint32_t bw = q == 0 ? wb[j].x : q == 1 ? wb[j].y : q == 2 ? wb[j].z : wb[j].w;
                    b = fmaf(__uint_as_float(bw << 16), xf.x, b);
                    b = fmaf(__uint_as_float(bw & 0xffff0000u), xf.y, b);
                }
            }
        }
    }
}

// in_proj_a/b, conv1d x3, activate, l2norm x2, decay_gate, gate_sigmoid and the recurrence of one layer
// (src/launcher.s:832-844; models/.../deltanet/kernels.ls:4-14):
//   a,b   = in_proj_a/b . xn                       (bf16 rows, fp32 accumulate)
//   c     = silu(conv1d(qkv))                      (4 taps, inference/recur.ls:12-40)
//   q     = l2norm(c_q) / sqrt(128), k = l2norm(c_k), v = c_v     (per head)
//   g     = exp(-exp(A_log) softplus(a + dt_bias)), beta = sigmoid(b)
//   r_j = sum_i k_i S_ij;  d_j = beta (v_j - r_j);  S_ij <- g S_ij + k_i d_j;  o_j = sum_i S_ij(new) q_i
// The conv history is a ring of 4 slots indexed by position, so the units that share a key head can all read the
// three previous slots while one of them writes the current one.
// EXT_AB: the two gate dot products come from elsewhere (other teams of the block computed them meanwhile): wait_ab() then
// ab[0], ab[1]; pos = the token position (read once by the caller).
template <bool STANDALONE, bool EXT_AB, class Sync, class WaitAB>
__device__ __forceinline__ void deltanet_layer_unit(const lb_dn_layer_params& p, int h, int jb, int t, dn_unit_smem& sm, Sync sync, int pos_in,
                                                    const volatile float* ab, WaitAB wait_ab) {
    float (&ks)[DN_D] = sm.ks, (&qs)[DN_D] = sm.qs, (&vs)[DN_COLS] = sm.vs, (&red)[16] = sm.red;
    float (&part)[16][DN_COLS] = sm.part;
    const int gqa = p.HV / p.HK, kh = h / gqa;
    const int tj = t & 7, ti = t >> 3;
    const int j0 = jb * DN_COLS + tj * 4;
    const int QK = p.HK * DN_D, C = 2 * QK + p.HV * DN_D;
    float* S = p.state + (size_t)h * DN_D * DN_D;

    // the state slab does not depend on the previous kernel of this step: load it first
    float4 s[8];
#pragma unroll
    for (int rr = 0; rr < 8; ++rr) s[rr] = *reinterpret_cast<const float4*>(S + (size_t)(ti + 16 * rr) * DN_D + j0);

    if (STANDALONE) pdl_wait();
    const int pos = STANDALONE ? p.pos[0] : pos_in;
    // (the convolution's operands and the decay / beta dot products below share one trip to L2: no block barrier lies
    // between their loads)
    // causal depthwise conv (ring history) + SiLU on this head's q, k channels and this slab's v channels
    auto conv = [&](int c) {
        const float x = __ldcg(p.qkvz + c);
        float y = bf16_bits_to_f32(p.conv_w[c]) * x;
        y = fmaf(bf16_bits_to_f32(p.conv_w[C + c]), p.conv_ring[(size_t)((pos + 3) & 3) * C + c], y);
        y = fmaf(bf16_bits_to_f32(p.conv_w[2 * C + c]), p.conv_ring[(size_t)((pos + 2) & 3) * C + c], y);
        y = fmaf(bf16_bits_to_f32(p.conv_w[3 * C + c]), p.conv_ring[(size_t)((pos + 1) & 3) * C + c], y);
        return siluf_dev(y);
    };
    const int cq = kh * DN_D + t, ck = QK + kh * DN_D + t, cv = 2 * QK + h * DN_D + jb * DN_COLS + t;
    float qv = conv(cq), kv = conv(ck);
    if (t < DN_COLS) vs[t] = conv(cv);
    // one CTA per key head (and every CTA for its own v channels) records the current token
    if (h % gqa == 0 && jb == 0) {
        p.conv_ring[(size_t)(pos & 3) * C + cq] = __ldcg(p.qkvz + cq);
        p.conv_ring[(size_t)(pos & 3) * C + ck] = __ldcg(p.qkvz + ck);
    }
    if (t < DN_COLS) p.conv_ring[(size_t)(pos & 3) * C + cv] = __ldcg(p.qkvz + cv);
    // decay / beta projections: two 5120-long dot products per value head
    float a = 0.f, b = 0.f;
    if (!EXT_AB) dn_gate_dot<2>(p, p.proj_a + (size_t)h * p.hidden, p.proj_b + (size_t)h * p.hidden, t, a, b);
    float qn = qv * qv, kn = kv * kv;
    dn_unit_sum4(a, b, qn, kn, red, t, sync);
    if (EXT_AB) {
        wait_ab();
        a = ab[0];
        b = ab[1];
    }
    const float tt = a + bf16_bits_to_f32(p.dt_bias[h]);
    const float sp = tt > 20.f ? tt : log1pf(expf(tt));
    const float g = expf(-expf(p.a_log[h]) * sp);
    const float beta = 1.0f / (1.0f + expf(-b));

    qs[t] = qv * rsqrtf(qn) * 0.08838834764831845f; // l2norm then 1/sqrt(128)
    ks[t] = kv * rsqrtf(kn);
    sync();
    if (STANDALONE) pdl_launch_dependents();

    float4 r = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int rr = 0; rr < 8; ++rr) {
        const float kk = ks[ti + 16 * rr];
        r.x = fmaf(kk, s[rr].x, r.x); r.y = fmaf(kk, s[rr].y, r.y);
        r.z = fmaf(kk, s[rr].z, r.z); r.w = fmaf(kk, s[rr].w, r.w);
    }
    *reinterpret_cast<float4*>(&part[ti][tj * 4]) = r;
    sync();
    r = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const float4 q4 = *reinterpret_cast<const float4*>(&part[i][tj * 4]);
        r.x += q4.x; r.y += q4.y; r.z += q4.z; r.w += q4.w;
    }
    float4 d;
    d.x = beta * (vs[tj * 4 + 0] - r.x); d.y = beta * (vs[tj * 4 + 1] - r.y);
    d.z = beta * (vs[tj * 4 + 2] - r.z); d.w = beta * (vs[tj * 4 + 3] - r.w);
    float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int rr = 0; rr < 8; ++rr) {
        const float kk = ks[ti + 16 * rr], qq = qs[ti + 16 * rr];
        s[rr].x = fmaf(kk, d.x, g * s[rr].x); s[rr].y = fmaf(kk, d.y, g * s[rr].y);
        s[rr].z = fmaf(kk, d.z, g * s[rr].z); s[rr].w = fmaf(kk, d.w, g * s[rr].w);
        o.x = fmaf(s[rr].x, qq, o.x); o.y = fmaf(s[rr].y, qq, o.y);
        o.z = fmaf(s[rr].z, qq, o.z); o.w = fmaf(s[rr].w, qq, o.w);
        *reinterpret_cast<float4*>(S + (size_t)(ti + 16 * rr) * DN_D + j0) = s[rr];
    }
    sync();
    *reinterpret_cast<float4*>(&part[ti][tj * 4]) = o;
    sync();
    if (ti == 0) {
        o = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const float4 q4 = *reinterpret_cast<const float4*>(&part[i][tj * 4]);
            o.x += q4.x; o.y += q4.y; o.z += q4.z; o.w += q4.w;
        }
        *reinterpret_cast<float4*>(p.out + (size_t)h * DN_D + j0) = o;
    }
}
