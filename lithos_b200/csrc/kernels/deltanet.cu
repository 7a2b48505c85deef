// Gated DeltaNet single-token recurrence for sm_100a.
//
// Restates inference/deltanet_fused.ls:97-149 (and delta_update.ls:24-54):
//   r_j   = sum_i k_i S_ij                  (pre-update, un-decayed state)
//   d_j   = beta (v_j - r_j)
//   S_ij <- g S_ij + k_i d_j
//   o_j   = sum_i S_ij(new) q_i             [ * silu(z_j) when z is given ]
// with decay g = exp(-exp(A_log) softplus(a + dt_bias)), beta = sigmoid(b)
// (inference/decay_gate.ls:28-57, inference/recur.ls:45-55).
//
// The reference walks the 64 KB head state twice from global memory with one
// thread per column.  Columns j of a head are independent, so here a CTA owns
// a 32-column slab of one head and holds it in REGISTERS (128 threads x 32
// fp32): the state is read from HBM once and written once per step, and when
// n_steps > 1 it stays on chip for the whole run of steps.
#include "deltanet_core.cuh"

template <typename T> __device__ __forceinline__ float ld_as_f32(const T* p, size_t i);
template <> __device__ __forceinline__ float ld_as_f32<float>(const float* p, size_t i) { return p[i]; }
template <> __device__ __forceinline__ float ld_as_f32<__nv_bfloat16>(const __nv_bfloat16* p, size_t i) {
    return __bfloat162float(p[i]);
}

// n_steps consecutive tokens: q,k are [n_steps][HK][128], v (z, out) are
// [n_steps][HV][128], g and beta are [n_steps][HV].
template <typename T>
__device__ __forceinline__ void deltanet_body(const lb_deltanet_params& p, int n_steps) {
    __shared__ float ks[DN_D], qs[DN_D];
    __shared__ __align__(16) float part[16][DN_COLS];
    const int h = blockIdx.x, jb = blockIdx.y;
    const int kh = h / (p.HV / p.HK);
    const int t = threadIdx.x, tj = t & 7, ti = t >> 3;
    const int j0 = jb * DN_COLS + tj * 4;
    float* S = p.state + (size_t)h * DN_D * DN_D;

    pdl_wait();
    float4 s[8];
#pragma unroll
    for (int rr = 0; rr < 8; ++rr) s[rr] = *reinterpret_cast<const float4*>(S + (size_t)(ti + 16 * rr) * DN_D + j0);

    for (int step = 0; step < n_steps; ++step) {
        const T* q = reinterpret_cast<const T*>(p.q) + ((size_t)step * p.HK + kh) * DN_D;
        const T* k = reinterpret_cast<const T*>(p.k) + ((size_t)step * p.HK + kh) * DN_D;
        const T* v = reinterpret_cast<const T*>(p.v) + ((size_t)step * p.HV + h) * DN_D;
        __syncthreads(); // previous step's readers of ks/qs/part are done
        ks[t] = ld_as_f32<T>(k, t);
        qs[t] = ld_as_f32<T>(q, t);
        __syncthreads();
        const float g = p.g[(size_t)step * p.HV + h], beta = p.beta[(size_t)step * p.HV + h];

        // r = S^T k over this thread's 8 rows, then across the 16 row phases
        float4 r = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int rr = 0; rr < 8; ++rr) {
            const float kk = ks[ti + 16 * rr];
            r.x = fmaf(kk, s[rr].x, r.x);
            r.y = fmaf(kk, s[rr].y, r.y);
            r.z = fmaf(kk, s[rr].z, r.z);
            r.w = fmaf(kk, s[rr].w, r.w);
        }
        *reinterpret_cast<float4*>(&part[ti][tj * 4]) = r;
        __syncthreads();
        r = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const float4 a = *reinterpret_cast<const float4*>(&part[i][tj * 4]);
            r.x += a.x; r.y += a.y; r.z += a.z; r.w += a.w;
        }
        float4 d;
        d.x = beta * (ld_as_f32<T>(v, j0 + 0) - r.x);
        d.y = beta * (ld_as_f32<T>(v, j0 + 1) - r.y);
        d.z = beta * (ld_as_f32<T>(v, j0 + 2) - r.z);
        d.w = beta * (ld_as_f32<T>(v, j0 + 3) - r.w);

        // update + read-out from the new state
        float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int rr = 0; rr < 8; ++rr) {
            const float kk = ks[ti + 16 * rr], qq = qs[ti + 16 * rr];
            s[rr].x = fmaf(kk, d.x, g * s[rr].x);
            s[rr].y = fmaf(kk, d.y, g * s[rr].y);
            s[rr].z = fmaf(kk, d.z, g * s[rr].z);
            s[rr].w = fmaf(kk, d.w, g * s[rr].w);
            o.x = fmaf(s[rr].x, qq, o.x);
            o.y = fmaf(s[rr].y, qq, o.y);
            o.z = fmaf(s[rr].z, qq, o.z);
            o.w = fmaf(s[rr].w, qq, o.w);
        }
        __syncthreads(); // everyone has consumed part[] from the r reduction
        *reinterpret_cast<float4*>(&part[ti][tj * 4]) = o;
        __syncthreads();
        if (ti == 0) {
            o = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const float4 a = *reinterpret_cast<const float4*>(&part[i][tj * 4]);
                o.x += a.x; o.y += a.y; o.z += a.z; o.w += a.w;
            }
            const size_t oi = ((size_t)step * p.HV + h) * DN_D + j0;
            if (p.z) {
                const float4 z = *reinterpret_cast<const float4*>(p.z + oi);
                o.x *= siluf_dev(z.x); o.y *= siluf_dev(z.y); o.z *= siluf_dev(z.z); o.w *= siluf_dev(z.w);
            }
            *reinterpret_cast<float4*>(p.out + oi) = o;
        }
    }
    pdl_launch_dependents();
#pragma unroll
    for (int rr = 0; rr < 8; ++rr) *reinterpret_cast<float4*>(S + (size_t)(ti + 16 * rr) * DN_D + j0) = s[rr];
}

extern "C" __global__ void __launch_bounds__(DN_THREADS) deltanet_step_bf16(const __grid_constant__ lb_deltanet_params p,
                                                                            int n_steps) {
    deltanet_body<__nv_bfloat16>(p, n_steps);
}
extern "C" __global__ void __launch_bounds__(DN_THREADS) deltanet_step_f32(const __grid_constant__ lb_deltanet_params p,
                                                                           int n_steps) {
    deltanet_body<float>(p, n_steps);
}

// g = exp(-exp(A_log) softplus(a + dt_bias)), beta = sigmoid(b); natural log
// as in models/.../deltanet/unroll.ls (DecayGate: softplus = ln(1+e^x)).
extern "C" __global__ void decay_gate_beta(const __grid_constant__ lb_decay_params p) {
    pdl_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= p.n) return;
    const float t = p.a[i] + p.dt_bias[i];
    const float sp = t > 20.f ? t : log1pf(expf(t));
    p.g[i] = expf(-expf(p.a_log[i]) * sp);
    if (p.b && p.beta) p.beta[i] = 1.0f / (1.0f + expf(-p.b[i]));
}

// ---------------------------------------------------------------------------
// The whole DeltaNet mixer of one layer in ONE kernel: what the reference runs
// as in_proj_a/b, conv1d x3, activate, l2norm x2, decay_gate, gate_sigmoid and
// the recurrence (src/launcher.s:832-844; models/.../deltanet/kernels.ls:4-14):
//   a,b   = in_proj_a/b . xn                       (bf16 rows, fp32 accumulate)
//   c     = silu(conv1d(qkv))                      (4 taps, inference/recur.ls:12-40)
//   q     = l2norm(c_q) / sqrt(128), k = l2norm(c_k), v = c_v     (per head)
//   g     = exp(-exp(A_log) softplus(a + dt_bias)), beta = sigmoid(b)
//   state update + read-out as in deltanet_body above.
// CTA = (value head, 32-column slab).  The conv history is a ring of 4 slots
// indexed by position, so the CTAs that share a key head can all read the three
// previous slots while one of them writes the current one.
// ---------------------------------------------------------------------------
extern "C" __global__ void __launch_bounds__(DN_THREADS) deltanet_layer_fused(const __grid_constant__ lb_dn_layer_params p) {
    __shared__ dn_unit_smem sm;
    deltanet_layer_unit<true, false>(p, blockIdx.x, blockIdx.y, threadIdx.x, sm, [] { __syncthreads(); }, 0, nullptr, [] {});
}
