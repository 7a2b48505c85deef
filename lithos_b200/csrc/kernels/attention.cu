// GQA decode attention (split-KV flash-decode) for sm_100a.
//
// Restates inference/attend.ls:85-191 (online-softmax loop over the KV cache,
// GQA map kv = h*n_kv/n_q, cache layout [seq, n_kv, d]) with the natural-exp
// soft-max and true -inf start of inference/attend_full.ls:186-196, and fuses
// what the reference runs as separate launches around it: per-head RMSNorm of
// q and of the new k (models/.../attention/kernels.ls:7-8), partial RoPE on
// interleaved pairs (inference/attend.ls:21-71), the KV append
// (src/launcher.s:2150-2247) and the sigmoid output gate
// (inference/attend_full.ls:236-248).
//
// The reference runs one CTA per query head and walks the positions serially
// with two barriers each.  Here a CTA owns one KV head and one slice of the
// positions, serves all G = HQ/HKV query heads of that KV head from a single
// pass over the bf16 K/V rows (KV bytes are the roofline), keeps a per-warp
// online soft-max, and the slices are merged in a fixed order by the last CTA
// to arrive (ordered, so run-to-run identical).
#include "attention_core.cuh"

template <int G>
__device__ __forceinline__ void attn_body(const lb_attn_params& p0, float* sm) {
    lb_attn_params p = p0;
    const int kv = blockIdx.x, split = blockIdx.y;
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    float* q_s = sm;                      // [G][256]
    float* kn_s = q_s + G * AT_D;         // [256] new key (bf16-rounded)
    float* vn_s = kn_s + AT_D;            // [256] new value (bf16-rounded)
    float* red = vn_s + AT_D;             // [40]
    float* wm = red + 40;                 // [8][G] per-warp max
    float* wl = wm + AT_WARPS * AT_GMAX;  // [8][G] per-warp sum
    float* wacc = wl + AT_WARPS * AT_GMAX; // [8][G][256]
    __shared__ uint32_t s_ticket;

    pdl_wait();
    if (p.pos_ptr) p.pos = p.pos_ptr[0];
    if (p.max_ctx > 0 && (p.pos < 0 || p.pos >= p.max_ctx)) { // the position lies outside the caches: report it, touch nothing
        if (threadIdx.x == 0 && blockIdx.x == 0 && blockIdx.y == 0 && p.status) atomicExch(p.status, LB_DEV_POS_RANGE);
        return;
    }
    const bool last = split == p.splits - 1;
    const float LOG2E = 1.4426950408889634f;
    const float qscale = rsqrtf((float)AT_D) * LOG2E; // scores kept in log2 units
    // cos/sin of this position once per CTA.  The angle pos*freq reaches 1e5 rad, far beyond fp32
    // resolution: it is formed and reduced modulo 2*pi in double (4 double operations), the
    // trigonometry itself is fp32 on |r| <= pi.  freq comes from the host in double.
    float* cs_s = wacc;       // the per-warp accumulators are not in use yet
    float* sn_s = wacc + 128;
    if (t < p.rot_dims / 2) {
        const double a = (double)p.pos * p.rope_freq[t];
        const double k = rint(a * 0.15915494309189535);
        const float r = (float)fma(-k, 6.283185307179586, a);
        sincosf(r, &sn_s[t], &cs_s[t]);
    }
    __syncthreads();
    for (int row = warp; row < G + (last ? 1 : 0); row += AT_WARPS) {
        if (row < G)
            warp_norm_rope(p.q, (size_t)(kv * G + row) * p.q_stride, p.in_dtype, p.q_norm_w, q_s + row * AT_D, cs_s, sn_s,
                           p.rot_dims, p.eps, qscale);
        else
            warp_norm_rope(p.k_new, (size_t)kv * AT_D, p.in_dtype, p.k_norm_w, kn_s, cs_s, sn_s, p.rot_dims, p.eps, 1.0f);
    }
    __syncthreads();
    if (last) {
        __nv_bfloat16 kb = __float2bfloat16_rn(kn_s[t]);
        __nv_bfloat16 vb = __float2bfloat16_rn(ld_in(p.v_new, (size_t)kv * AT_D + t, p.in_dtype));
        const size_t row = ((size_t)p.pos * p.HKV + kv) * AT_D + t;
        reinterpret_cast<__nv_bfloat16*>(p.k_cache)[row] = kb; // KV append
        reinterpret_cast<__nv_bfloat16*>(p.v_cache)[row] = vb;
        kn_s[t] = __bfloat162float(kb);
        vn_s[t] = __bfloat162float(vb);
    }
    __syncthreads();
    pdl_launch_dependents();

    // the query heads stay in shared memory (two 128-bit loads per head and row): registers hold
    // the running soft-max state only, so that two CTAs fit on an SM
    const float4* q4 = reinterpret_cast<const float4*>(q_s) + lane * 2;

    float m[G], l[G], acc[G][8];
#pragma unroll
    for (int g = 0; g < G; ++g) {
        m[g] = -INFINITY;
        l[g] = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[g][j] = 0.f;
    }

    const int chunk = (p.pos + p.splits - 1) / p.splits;
    const int t0 = split * chunk, t1 = min(p.pos, t0 + chunk);
    const size_t row_stride = (size_t)p.HKV * AT_D;
    const uint4* kbase = reinterpret_cast<const uint4*>(p.k_cache + (size_t)kv * AT_D) + lane;
    const uint4* vbase = reinterpret_cast<const uint4*>(p.v_cache + (size_t)kv * AT_D) + lane;

    auto step = [&](const float (&kf)[8], const float (&vf)[8]) {
        float s[G];
#pragma unroll
        for (int g = 0; g < G; ++g) {
            const float4 qa = q4[g * (AT_D / 4)], qb = q4[g * (AT_D / 4) + 1];
            float d = qa.x * kf[0];
            d = fmaf(qa.y, kf[1], d); d = fmaf(qa.z, kf[2], d); d = fmaf(qa.w, kf[3], d);
            d = fmaf(qb.x, kf[4], d); d = fmaf(qb.y, kf[5], d); d = fmaf(qb.z, kf[6], d); d = fmaf(qb.w, kf[7], d);
            s[g] = d;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
#pragma unroll
            for (int g = 0; g < G; ++g) s[g] += __shfl_xor_sync(0xffffffffu, s[g], o);
#pragma unroll
        for (int g = 0; g < G; ++g) {
            const float mn = fmaxf(m[g], s[g]);
            const float corr = exp2f(m[g] - mn); // exp2f(-inf) = 0 on the first row
            const float pr = exp2f(s[g] - mn);
            m[g] = mn;
            l[g] = fmaf(l[g], corr, pr);
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[g][j] = fmaf(acc[g][j], corr, pr * vf[j]);
        }
    };
    auto unpack = [](const uint4& raw, float (&f)[8]) {
        f[0] = __uint_as_float(raw.x << 16); f[1] = __uint_as_float(raw.x & 0xffff0000u);
        f[2] = __uint_as_float(raw.y << 16); f[3] = __uint_as_float(raw.y & 0xffff0000u);
        f[4] = __uint_as_float(raw.z << 16); f[5] = __uint_as_float(raw.z & 0xffff0000u);
        f[6] = __uint_as_float(raw.w << 16); f[7] = __uint_as_float(raw.w & 0xffff0000u);
    };

    int r = t0 + warp;
    // two rows in flight per warp
    for (; r + AT_WARPS < t1; r += 2 * AT_WARPS) {
        uint4 k0 = __ldg(kbase + (size_t)r * (row_stride / 8));
        uint4 v0 = __ldg(vbase + (size_t)r * (row_stride / 8));
        uint4 k1 = __ldg(kbase + (size_t)(r + AT_WARPS) * (row_stride / 8));
        uint4 v1 = __ldg(vbase + (size_t)(r + AT_WARPS) * (row_stride / 8));
        float kf[8], vf[8];
        unpack(k0, kf); unpack(v0, vf); step(kf, vf);
        unpack(k1, kf); unpack(v1, vf); step(kf, vf);
    }
    for (; r < t1; r += AT_WARPS) {
        uint4 k0 = __ldg(kbase + (size_t)r * (row_stride / 8));
        uint4 v0 = __ldg(vbase + (size_t)r * (row_stride / 8));
        float kf[8], vf[8];
        unpack(k0, kf); unpack(v0, vf); step(kf, vf);
    }
    if (last && warp == 0) { // the token being decoded, straight from shared memory
        float kf[8], vf[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            kf[j] = kn_s[lane * 8 + j];
            vf[j] = vn_s[lane * 8 + j];
        }
        step(kf, vf);
    }

    // ---- merge the 8 warps (fixed order) ----
#pragma unroll
    for (int g = 0; g < G; ++g) {
        if (lane == 0) {
            wm[warp * AT_GMAX + g] = m[g];
            wl[warp * AT_GMAX + g] = l[g];
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) wacc[((size_t)warp * G + g) * AT_D + lane * 8 + j] = acc[g][j];
    }
    __syncthreads();
    float Mg[G], Lg[G], Ag[G]; // thread t owns dim t
#pragma unroll
    for (int g = 0; g < G; ++g) {
        float M = -INFINITY;
        for (int w = 0; w < AT_WARPS; ++w) M = fmaxf(M, wm[w * AT_GMAX + g]);
        float L = 0.f, A = 0.f;
        for (int w = 0; w < AT_WARPS; ++w) {
            const float mw = wm[w * AT_GMAX + g];
            const float sc = mw == -INFINITY ? 0.f : exp2f(mw - M);
            L = fmaf(wl[w * AT_GMAX + g], sc, L);
            A = fmaf(wacc[((size_t)w * G + g) * AT_D + t], sc, A);
        }
        Mg[g] = M; Lg[g] = L; Ag[g] = A;
    }

    // ---- merge the position slices across CTAs (fixed order, last arriver) ----
    if (p.splits > 1) {
        float* rec = p.scratch + ((size_t)(kv * p.splits + split) * G) * AT_REC;
#pragma unroll
        for (int g = 0; g < G; ++g) {
            __stcg(rec + g * AT_REC + t, Ag[g]);
            if (t == 0) {
                __stcg(rec + g * AT_REC + 256, Mg[g]);
                __stcg(rec + g * AT_REC + 257, Lg[g]);
            }
        }
        __threadfence();
        __syncthreads();
        if (t == 0) s_ticket = atomicAdd(p.counters + kv, 1u);
        __syncthreads();
        if (s_ticket != (uint32_t)(p.splits - 1)) return;
        __threadfence();
        // all (max, sum) pairs of this KV head in one parallel pass, then the slice weights once
        float* ms_s = wacc;                       // [splits][G] slice maxima, then slice weights
        float* ls_s = wacc + p.splits * G;        // [splits][G] slice sums
        float* Mx_s = wacc + 2 * p.splits * G;    // [G]
        const float* kvrec = p.scratch + (size_t)kv * p.splits * G * AT_REC;
        for (int i = t; i < p.splits * G; i += AT_THREADS) {
            ms_s[i] = __ldcg(kvrec + (size_t)i * AT_REC + 256);
            ls_s[i] = __ldcg(kvrec + (size_t)i * AT_REC + 257);
        }
        __syncthreads();
        if (t < G) {
            float M = -INFINITY;
            for (int s2 = 0; s2 < p.splits; ++s2) M = fmaxf(M, ms_s[s2 * G + t]);
            Mx_s[t] = M;
        }
        __syncthreads();
        for (int i = t; i < p.splits * G; i += AT_THREADS) {
            const float mi = ms_s[i];
            ms_s[i] = mi == -INFINITY ? 0.f : exp2f(mi - Mx_s[i % G]);
        }
        __syncthreads();
#pragma unroll
        for (int g = 0; g < G; ++g) { Lg[g] = 0.f; Ag[g] = 0.f; }
        int s2 = 0;
        for (; s2 + 8 <= p.splits; s2 += 8) { // 8*G independent loads in flight, then added in slice order
            float a8[G][8];
#pragma unroll
            for (int g = 0; g < G; ++g)
#pragma unroll
                for (int j = 0; j < 8; ++j) a8[g][j] = __ldcg(kvrec + ((size_t)(s2 + j) * G + g) * AT_REC + t);
#pragma unroll
            for (int g = 0; g < G; ++g)
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const float w = ms_s[(s2 + j) * G + g];
                    Lg[g] = fmaf(ls_s[(s2 + j) * G + g], w, Lg[g]);
                    Ag[g] = fmaf(a8[g][j], w, Ag[g]);
                }
        }
        for (; s2 < p.splits; ++s2)
#pragma unroll
            for (int g = 0; g < G; ++g) {
                const float w = ms_s[s2 * G + g];
                Lg[g] = fmaf(ls_s[s2 * G + g], w, Lg[g]);
                Ag[g] = fmaf(__ldcg(kvrec + ((size_t)s2 * G + g) * AT_REC + t), w, Ag[g]);
            }
        if (t == 0) p.counters[kv] = 0u;
    }
#pragma unroll
    for (int g = 0; g < G; ++g) {
        const int hq = kv * G + g;
        float o = Ag[g] / Lg[g];
        if (p.gate) o *= sigmoidf_dev(ld_in(p.gate, (size_t)hq * p.gate_stride + t, p.in_dtype));
        p.out[(size_t)hq * AT_D + t] = o;
    }
}

extern "C" __global__ void __launch_bounds__(AT_THREADS, 2) attn_decode_split(const __grid_constant__ lb_attn_params p) {
    extern __shared__ __align__(16) float at_sm[];
    const int G = p.HQ / p.HKV;
    switch (G) {
        case 1: attn_body<1>(p, at_sm); break;
        case 2: attn_body<2>(p, at_sm); break;
        case 3: attn_body<3>(p, at_sm); break;
        case 4: attn_body<4>(p, at_sm); break;
        case 6: attn_body<6>(p, at_sm); break;
        default: break; // host rejects other ratios
    }
}
