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

// Thread (column jl of the slab, row quarter q4 = t & 3) holds rows 32*q4 .. 32*q4+31 of its column: the sums over rows
// are 32 local terms and two shuffles between the four neighbouring lanes of a column, no shared-memory reduction.  With
// the state on chip a step is a chain of latencies (one warp per scheduler) shorter than a trip to L2, so the operands of
// a step (k, q, the slab's 32 values of v, g, beta) are copied DN_AHEAD - 1 steps ahead into a ring in shared memory by
// cp.async -- loads into registers that far ahead still stalled every step, because a warp waits on a scoreboard counter,
// not on one load -- and a step costs one block barrier.
#define DN_AHEAD 4
template <typename T> struct dn_in; // element type of q, k, v: how four consecutive values read as fp32
template <> struct dn_in<float> {
    static __device__ __forceinline__ float4 ld4(const unsigned char* p) { return *reinterpret_cast<const float4*>(p); }
    static __device__ __forceinline__ float ld1(const unsigned char* p) { return *reinterpret_cast<const float*>(p); }
};
template <> struct dn_in<__nv_bfloat16> {
    static __device__ __forceinline__ float4 ld4(const unsigned char* p) {
        const uint2 u = *reinterpret_cast<const uint2*>(p);
        return make_float4(__uint_as_float(u.x << 16), __uint_as_float(u.x & 0xffff0000u), __uint_as_float(u.y << 16), __uint_as_float(u.y & 0xffff0000u));
    }
    static __device__ __forceinline__ float ld1(const unsigned char* p) { return __uint_as_float((uint32_t)*reinterpret_cast<const uint16_t*>(p) << 16); }
};
__device__ __forceinline__ void dn_cp16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void dn_cp4(void* dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}

// n_steps consecutive tokens: q,k are [n_steps][HK][128], v (z, out) are
// [n_steps][HV][128], g and beta are [n_steps][HV].
template <typename T>
__device__ __forceinline__ void deltanet_body(const lb_deltanet_params& p, int n_steps) {
    constexpr int E = (int)sizeof(T);
    constexpr int QS = 32 * E + 16;        // bytes per row quarter of k / q in a stage (+16: the four quarters on different banks)
    constexpr int CQ = 2 * E;              // 16-byte pieces per row quarter
    constexpr int OFF_Q = 4 * QS, OFF_V = 8 * QS, OFF_G = OFF_V + 32 * E, STAGE = OFF_G + 16;
    __shared__ __align__(16) unsigned char ring[DN_AHEAD][STAGE];
    const int h = blockIdx.x, jb = blockIdx.y;
    const int kh = h / (p.HV / p.HK);
    const int t = threadIdx.x, q4 = t & 3, jl = t >> 2;
    const int j = jb * DN_COLS + jl;
    float* S = p.state + (size_t)h * DN_D * DN_D + (size_t)(32 * q4) * DN_D + j;

    pdl_wait();
    // every thread brings at most one piece of a step's operands: 4 CQ pieces of k, 4 CQ of q, 2 E of v, g, beta
    auto fetch = [&](int step) {
        unsigned char* st = ring[step % DN_AHEAD];
        if (t < 8 * CQ) {
            const int which = t / (4 * CQ), i = t % (4 * CQ); // k or q, piece i of its 128 values
            const unsigned char* src = reinterpret_cast<const unsigned char*>(which ? p.q : p.k) + ((size_t)step * p.HK + kh) * DN_D * E;
            dn_cp16(st + which * OFF_Q + (i / CQ) * QS + (i % CQ) * 16, src + i * 16);
        } else if (t < 8 * CQ + 2 * E) {
            const int i = t - 8 * CQ;
            dn_cp16(st + OFF_V + i * 16, reinterpret_cast<const unsigned char*>(p.v) + (((size_t)step * p.HV + h) * DN_D + jb * DN_COLS) * E + i * 16);
        } else if (t == 8 * CQ + 2 * E) {
            dn_cp4(st + OFF_G, p.g + (size_t)step * p.HV + h);
        } else if (t == 8 * CQ + 2 * E + 1) {
            dn_cp4(st + OFF_G + 4, p.beta + (size_t)step * p.HV + h);
        }
    };
#pragma unroll
    for (int u = 0; u < DN_AHEAD - 1; ++u) {
        if (u < n_steps) fetch(u);
        asm volatile("cp.async.commit_group;" ::: "memory"); // one group per step, empty or not: the wait below counts groups
    }
    float s[32];
#pragma unroll
    for (int rr = 0; rr < 32; ++rr) s[rr] = S[(size_t)rr * DN_D];

    for (int step = 0; step < n_steps; ++step) {
        asm volatile("cp.async.wait_group %0;" ::"n"(DN_AHEAD - 2) : "memory"); // this thread's piece of this step has landed
        __syncthreads(); // everybody's pieces are visible, and everybody is done with the previous step's stage ...
        if (step + DN_AHEAD - 1 < n_steps) fetch(step + DN_AHEAD - 1); // ... which the step DN_AHEAD - 1 ahead now takes
        asm volatile("cp.async.commit_group;" ::: "memory");
        const unsigned char* st = ring[step % DN_AHEAD];
        const unsigned char* kq = st + q4 * QS;
        const float g = *reinterpret_cast<const float*>(st + OFF_G), beta = *reinterpret_cast<const float*>(st + OFF_G + 4);
        const float v = dn_in<T>::ld1(st + OFF_V + jl * E);

        // r_j = sum_i k_i S_ij (pre-update state): four running sums per thread, then the column's four lanes
        float r0 = 0.f, r1 = 0.f, r2 = 0.f, r3 = 0.f;
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            const float4 kk = dn_in<T>::ld4(kq + c * 4 * E);
            r0 = fmaf(kk.x, s[4 * c + 0], r0);
            r1 = fmaf(kk.y, s[4 * c + 1], r1);
            r2 = fmaf(kk.z, s[4 * c + 2], r2);
            r3 = fmaf(kk.w, s[4 * c + 3], r3);
        }
        float r = (r0 + r1) + (r2 + r3);
        r += __shfl_xor_sync(0xffffffffu, r, 1);
        r += __shfl_xor_sync(0xffffffffu, r, 2);
        const float d = beta * (v - r);

        // S_ij <- g S_ij + k_i d_j, o_j = sum_i S_ij(new) q_i
        float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            const float4 kk = dn_in<T>::ld4(kq + c * 4 * E), qq = dn_in<T>::ld4(kq + OFF_Q + c * 4 * E);
            s[4 * c + 0] = fmaf(kk.x, d, g * s[4 * c + 0]);
            s[4 * c + 1] = fmaf(kk.y, d, g * s[4 * c + 1]);
            s[4 * c + 2] = fmaf(kk.z, d, g * s[4 * c + 2]);
            s[4 * c + 3] = fmaf(kk.w, d, g * s[4 * c + 3]);
            o0 = fmaf(s[4 * c + 0], qq.x, o0);
            o1 = fmaf(s[4 * c + 1], qq.y, o1);
            o2 = fmaf(s[4 * c + 2], qq.z, o2);
            o3 = fmaf(s[4 * c + 3], qq.w, o3);
        }
        float o = (o0 + o1) + (o2 + o3);
        o += __shfl_xor_sync(0xffffffffu, o, 1);
        o += __shfl_xor_sync(0xffffffffu, o, 2);
        if (q4 == 0) {
            const size_t oi = ((size_t)step * p.HV + h) * DN_D + j;
            if (p.z) o *= siluf_dev(p.z[oi]);
            p.out[oi] = o;
        }
    }
    pdl_launch_dependents();
#pragma unroll
    for (int rr = 0; rr < 32; ++rr) S[(size_t)rr * DN_D] = s[rr];
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
