// GPTQ int4 weight-only GEMV for batch-1 decode on sm_100a.
//
// Replaces the reference's minds/gptq_gemv_safe.ptx (and its v2..v9 siblings,
// inference/gemv.ls) for the primary contract: qweight int32 [K/8,N] (nibble j
// of word (kp,n) is k = 8kp+j), scales fp16 [K/128,N], qzeros int32
// [K/128,N/8] (NULL = zero-point 8, the reference's constant), x fp16, fp32
// accumulation over groups, y fp16/fp32.
//
// Shape of the kernel (HBM-bound, ~0.5 B/weight):
//   * CTA (tile, split) owns 128 output columns and a contiguous range of
//     K-groups.  One elected producer lane streams "units" (half a group: a box
//     of 8 packed rows x 512 B) into a ring of shared-memory stages with one
//     tiled TMA load each (cp.async.bulk.tensor.2d, completion on an mbarrier,
//     L2 evict-first hint since weights are read once).
//   * 8 consumer warps each take whole units round-robin; a lane owns 4
//     adjacent columns (one 128-bit shared load per packed row) and fetches its
//     4 scales / zero-points of the unit's group straight from global memory.
//   * Dequant in registers: (word & 0x000f000f) | 0x6400 6400 is the fp16x2
//     pair (1024+q_j, 1024+q_{j+4}); one HSUB2/HFMA2 turns it into exact
//     integers (q-8); four HFMA2 against the matching x pairs give the
//     8-weight partial dot product, widened to fp32 once per packed word.
//     The per-group scale and the zero-point correction (8-z)*sum(x) are
//     applied once per unit in fp32.
//   * Reduction is ordered everywhere (warp order inside the CTA, split order
//     across CTAs through a scratch buffer and a self-resetting arrival
//     counter), so results are bit-identical run to run; the reference's
//     atom.global.add.f32 split-K is not reproduced.
//   * The producer starts prefetching weights before griddepcontrol.wait, so
//     under programmatic dependent launch the copy pipeline is already full
//     when the previous kernel's output (x) becomes visible.
#include "common.cuh"
#include "params.h"

#define CONSUMERS (LB_GEMV_WARPS * 32)
#define UROWS LB_GEMV_UNIT_ROWS

__device__ __forceinline__ void consumer_bar() { asm volatile("bar.sync 1, %0;" ::"n"(CONSUMERS) : "memory"); }

__device__ __forceinline__ uint32_t lop3_and_or(uint32_t a, uint32_t mask, uint32_t magic) {
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(a), "r"(mask), "r"(magic)); // (a & mask) | magic
    return r;
}

// One tiled TMA load: box (UROWS rows x 128 columns of packed words) at
// (column x, packed row y) of the qweight matrix into one shared-memory stage.
__device__ __forceinline__ void tma_load_box(void* dst_smem, const void* tmap, int x, int y, uint64_t* bar, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint"
        " [%0], [%1, {%2, %3}], [%4], %5;" ::"r"(smem_u32(dst_smem)),
        "l"(tmap), "r"(x), "r"(y), "r"(smem_u32(bar)), "l"(policy)
        : "memory");
}

// partial dot product of one packed word (8 weights of one column, zero-point
// 8 removed) with the 8 matching activations; returns fp32
__device__ __forceinline__ float dot8(uint32_t w, const __half2 (&xp)[4]) {
    const uint32_t MAGIC = 0x64006400u;                        // fp16x2 (1024, 1024)
    const __half2 BIAS_LO = __halves2half2(__ushort_as_half(0x6408), __ushort_as_half(0x6408)); // 1032
    const __half2 SIXTEENTH = __halves2half2(__ushort_as_half(0x2C00), __ushort_as_half(0x2C00)); // 1/16
    const __half2 BIAS_HI = __halves2half2(__ushort_as_half(0xD480), __ushort_as_half(0xD480));   // -72
    uint32_t w8 = w >> 8;
    uint32_t a = lop3_and_or(w, 0x000f000fu, MAGIC);   // 1024 + (q0, q4)
    uint32_t b = lop3_and_or(w, 0x00f000f0u, MAGIC);   // 1024 + 16*(q1, q5)
    uint32_t c = lop3_and_or(w8, 0x000f000fu, MAGIC);  // 1024 + (q2, q6)
    uint32_t d = lop3_and_or(w8, 0x00f000f0u, MAGIC);  // 1024 + 16*(q3, q7)
    __half2 qa = __hsub2(*reinterpret_cast<__half2*>(&a), BIAS_LO);
    __half2 qb = __hfma2(*reinterpret_cast<__half2*>(&b), SIXTEENTH, BIAS_HI);
    __half2 qc = __hsub2(*reinterpret_cast<__half2*>(&c), BIAS_LO);
    __half2 qd = __hfma2(*reinterpret_cast<__half2*>(&d), SIXTEENTH, BIAS_HI);
    __half2 p = __hmul2(qa, xp[0]);
    p = __hfma2(qb, xp[1], p);
    p = __hfma2(qc, xp[2], p);
    p = __hfma2(qd, xp[3], p);
    float2 f = __half22float2(p);
    return f.x + f.y;
}

extern "C" __global__ void __launch_bounds__(CONSUMERS + 32, 2) gemv_int4_w128(const __grid_constant__ lb_gemv_params p) {
    extern __shared__ __align__(128) unsigned char smem[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int tile = blockIdx.x, split = blockIdx.y;
    const int n0 = tile * LB_GEMV_TILE_N;
    const int ncols = min(LB_GEMV_TILE_N, p.N - n0);
    const int groups = p.K / LB_GEMV_GROUP;
    const int g0 = split * p.groups_per_split;
    const int g1 = min(groups, g0 + p.groups_per_split);
    const int n_units = max(0, g1 - g0) * (LB_GEMV_ROWS / UROWS); // half-group units
    const int S = p.stages;

    // shared-memory carve-up
    unsigned char* stage_base = smem;
    uint4* xs = reinterpret_cast<uint4*>(smem + (size_t)S * LB_GEMV_STAGE_BYTES);           // [rows] permuted fp16 x
    float* xsum = reinterpret_cast<float*>(xs + (size_t)p.groups_per_split * LB_GEMV_ROWS); // [units]
    float* red = xsum + ((2 * p.groups_per_split + 3) & ~3);                                // [8][128] + 40
    uint64_t* full = reinterpret_cast<uint64_t*>(red + LB_GEMV_WARPS * LB_GEMV_TILE_N + 40);
    uint64_t* empty = full + S;
    __shared__ uint32_t s_ticket;
    __shared__ uint32_t s_bad;

    if (tid == 0) {
        for (int s = 0; s < S; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        s_bad = 0;
        mbar_fence_init();
    }
    __syncthreads();

    if (warp == LB_GEMV_WARPS) {
        // ---------------- producer: one elected lane streams boxes into the ring ----------------
        // Weights never change, so this starts before griddepcontrol.wait: under programmatic
        // dependent launch the ring is already full when the activations become visible.
        if (lane == 0) {
            const uint64_t pol = l2_policy_evict_first();
            const int row0 = g0 * LB_GEMV_ROWS;
            for (int u = 0; u < n_units; ++u) {
                const int s = u % S;
                if (u >= S && !mbar_wait(&empty[s], ((u / S) - 1) & 1)) {
                    atomicExch(p.status, LB_DEV_TIMEOUT_EMPTY);
                    s_bad = 1;
                    break;
                }
                mbar_arrive_expect_tx(&full[s], LB_GEMV_STAGE_BYTES);
                tma_load_box(stage_base + (size_t)s * LB_GEMV_STAGE_BYTES, p.tmap, n0, row0 + u * UROWS, &full[s], pol);
            }
        }
        return; // consumers wait for every box, so no copy is in flight when the CTA ends
    }

    // ---------------- consumer warps ----------------
    pdl_wait(); // x (and y for accumulate mode) come from the previous kernel

    const int rows = n_units * UROWS;
    const int row0 = g0 * LB_GEMV_ROWS; // first packed row of this split

    // --- prologue: build the fp16 activation slice in shared memory ---
    float rinv = 1.0f;
    if (p.x_mode == LB_X_F32_RMSNORM) {
        const float4* xv = reinterpret_cast<const float4*>(p.x);
        float ss = 0.f;
        for (int i = tid; i < p.K / 4; i += CONSUMERS) {
            float4 v = __ldg(xv + i);
            ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        }
        ss = warp_sum(ss);
        if (lane == 0) red[warp] = ss;
        consumer_bar();
        float tot = 0.f;
#pragma unroll
        for (int w = 0; w < LB_GEMV_WARPS; ++w) tot += red[w];
        rinv = rsqrtf(tot / (float)p.K + p.eps);
        consumer_bar();
    }
    for (int rb = 0; rb < rows; rb += CONSUMERS) {
        const int r = rb + tid;         // row within the split (16-lane segments never straddle a group)
        const bool live = r < rows;
        const int k = (row0 + r) * 8;   // first k of this packed row
        float v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = 0.f;
        if (live) {
            if (p.x_mode == LB_X_F16) {
                uint4 raw = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const __half*>(p.x) + k));
                const __half2* h = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    float2 f = __half22float2(h[j]);
                    v[2 * j] = f.x;
                    v[2 * j + 1] = f.y;
                }
            } else {
                const float4* xv = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p.x) + k);
                float4 a = __ldg(xv), b = __ldg(xv + 1);
                v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
                v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
            }
        }
        if (p.x_mode == LB_X_F32_RMSNORM) {
            if (live) {
                uint4 wr = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(p.aux0) + k));
                const uint16_t* wb = reinterpret_cast<const uint16_t*>(&wr);
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] = v[j] * rinv * (1.0f + bf16_bits_to_f32(wb[j]));
            }
        } else if (p.x_mode == LB_X_F32_HEADNORM_SILU) {
            // one head = 128 values = the 16 rows held by a 16-lane segment
            float ss = 0.f;
#pragma unroll
            for (int j = 0; j < 8; ++j) ss += v[j] * v[j];
#pragma unroll
            for (int o = 8; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            float hr = rsqrtf(ss * (1.0f / 128.0f) + p.eps);
            if (live) {
                const float4* zv = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p.aux1) + k);
                const float4* wv = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p.aux0) + (k & 127));
                float4 za = __ldg(zv), zb = __ldg(zv + 1), wa = __ldg(wv), wb = __ldg(wv + 1);
                float z[8] = {za.x, za.y, za.z, za.w, zb.x, zb.y, zb.z, zb.w};
                float w[8] = {wa.x, wa.y, wa.z, wa.w, wb.x, wb.y, wb.z, wb.w};
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] = v[j] * hr * w[j] * siluf_dev(z[j]);
            }
        }
        __half h[8];
        float rs = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            h[j] = __float2half_rn(v[j]);
            rs += __half2float(h[j]);
        }
        // sum over the 8 rows of the unit (8-lane segment)
#pragma unroll
        for (int o = 4; o > 0; o >>= 1) rs += __shfl_xor_sync(0xffffffffu, rs, o);
        if (live) {
            __half2 pr[4] = {__halves2half2(h[0], h[4]), __halves2half2(h[1], h[5]), __halves2half2(h[2], h[6]),
                             __halves2half2(h[3], h[7])};
            xs[r] = *reinterpret_cast<uint4*>(pr);
            if ((lane & 7) == 0) xsum[r >> 3] = rs;
            if (p.x_out && tile == 0) {
                __half2 pl[4] = {__halves2half2(h[0], h[1]), __halves2half2(h[2], h[3]), __halves2half2(h[4], h[5]),
                                 __halves2half2(h[6], h[7])};
                *reinterpret_cast<uint4*>(p.x_out + k) = *reinterpret_cast<uint4*>(pl);
            }
        }
    }
    consumer_bar();
    pdl_launch_dependents();

    // --- main loop: each warp consumes whole units; a lane owns 4 adjacent columns ---
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    const bool col_ok = lane * 4 < ncols;
    for (int u = warp; u < n_units; u += LB_GEMV_WARPS) {
        const int s = u % S;
        const int g = g0 + (u >> 1);
        // this unit's scales / zero-points for the lane's columns: issued first, used last
        uint2 sraw = make_uint2(0u, 0u);
        uint32_t zw = 0x88888888u;
        if (col_ok) {
            sraw = __ldg(reinterpret_cast<const uint2*>(p.scales + (size_t)g * p.N + n0 + lane * 4));
            if (p.qzeros) zw = __ldg(p.qzeros + (size_t)g * (p.N >> 3) + (n0 >> 3) + (lane >> 1));
        }
        if (!mbar_wait(&full[s], (u / S) & 1)) {
            if (lane == 0) { atomicExch(p.status, LB_DEV_TIMEOUT_FULL); s_bad = 1; }
            break;
        }
        const unsigned char* st = stage_base + (size_t)s * LB_GEMV_STAGE_BYTES;
        float ga[4] = {0.f, 0.f, 0.f, 0.f};
        const uint4* xrow = xs + u * UROWS;
#pragma unroll
        for (int r = 0; r < UROWS; ++r) {
            uint4 w = *reinterpret_cast<const uint4*>(st + r * (LB_GEMV_TILE_N * 4) + lane * 16);
            uint4 xr = xrow[r];
            const __half2(&xp)[4] = *reinterpret_cast<const __half2(*)[4]>(&xr);
            ga[0] += dot8(w.x, xp);
            ga[1] += dot8(w.y, xp);
            ga[2] += dot8(w.z, xp);
            ga[3] += dot8(w.w, xp);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[s]); // stage may be refilled
        float2 s01 = __half22float2(*reinterpret_cast<__half2*>(&sraw.x));
        float2 s23 = __half22float2(*reinterpret_cast<__half2*>(&sraw.y));
        zw >>= (lane & 1) * 16;
        const float xsu = xsum[u];
        acc[0] = fmaf(s01.x, fmaf(8.0f - (float)(zw & 0xFu), xsu, ga[0]), acc[0]);
        acc[1] = fmaf(s01.y, fmaf(8.0f - (float)((zw >> 4) & 0xFu), xsu, ga[1]), acc[1]);
        acc[2] = fmaf(s23.x, fmaf(8.0f - (float)((zw >> 8) & 0xFu), xsu, ga[2]), acc[2]);
        acc[3] = fmaf(s23.y, fmaf(8.0f - (float)((zw >> 12) & 0xFu), xsu, ga[3]), acc[3]);
    }

    // --- ordered reduction across the 8 warps ---
    *reinterpret_cast<float4*>(red + warp * LB_GEMV_TILE_N + lane * 4) = make_float4(acc[0], acc[1], acc[2], acc[3]);
    consumer_bar();
    float v = 0.f;
    if (tid < LB_GEMV_TILE_N) {
#pragma unroll
        for (int w = 0; w < LB_GEMV_WARPS; ++w) v += red[w * LB_GEMV_TILE_N + tid];
    }

    // --- ordered split-K across CTAs: last arriver sums the partials ---
    if (p.ksplit > 1) {
        if (tid < ncols) __stcg(p.partial + (size_t)split * p.N + n0 + tid, v);
        __threadfence();
        consumer_bar();
        if (tid == 0) s_ticket = atomicAdd(p.counters + tile, 1u);
        consumer_bar();
        if (s_ticket != (uint32_t)(p.ksplit - 1)) return;
        __threadfence();
        v = 0.f;
        if (tid < ncols)
            for (int sp = 0; sp < p.ksplit; ++sp) v += __ldcg(p.partial + (size_t)sp * p.N + n0 + tid);
        if (tid == 0) p.counters[tile] = 0u; // ready for the next launch on this stream
    }

    // --- epilogue ---
    if (s_bad) return;
    if (p.y_mode == LB_Y_SWIGLU_F16) {
        consumer_bar(); // red is reused below; every warp has finished reading it
        if (tid < LB_GEMV_TILE_N) red[tid] = v;
        consumer_bar();
        if (tid < ncols / 2) {
            float gate = red[tid], up = red[tid + 64];
            reinterpret_cast<__half*>(p.y)[n0 / 2 + tid] = __float2half_rn(siluf_dev(gate) * up);
        }
        return;
    }
    if (tid < ncols) {
        const int n = n0 + tid;
        if (p.y_mode == LB_Y_F16) reinterpret_cast<__half*>(p.y)[n] = __float2half_rn(v);
        else if (p.y_mode == LB_Y_F32) reinterpret_cast<float*>(p.y)[n] = v;
        else reinterpret_cast<float*>(p.y)[n] += v;
    }
}

// ---------------------------------------------------------------------------
// Dequantisation and unpack as stand-alone kernels: the bit-exact targets of
// the parity tests, and the weight path of the batched (tensor-core) GEMM.
// W(k,n) = fma(float(q), s, -z*s) exactly as minds/gptq_gemv_safe.ptx:221-262.
// ---------------------------------------------------------------------------
extern "C" __global__ void gptq_dequant_f32(const uint32_t* __restrict__ qweight, const __half* __restrict__ scales,
                                            const uint32_t* __restrict__ qzeros, float* __restrict__ w_out, int K,
                                            int N) {
    const int n = blockIdx.x * blockDim.x + threadIdx.x;
    const int kp = blockIdx.y;
    if (n >= N || kp >= K / 8) return;
    const int g = kp >> 4;
    const uint32_t w = qweight[(size_t)kp * N + n];
    const float s = __half2float(scales[(size_t)g * N + n]);
    const uint32_t z = qzeros ? (qzeros[(size_t)g * (N / 8) + (n >> 3)] >> (4 * (n & 7))) & 0xFu : 8u;
    const float bias = -(float)z * s;
#pragma unroll
    for (int j = 0; j < 8; ++j) w_out[((size_t)kp * 8 + j) * N + n] = fmaf((float)((w >> (4 * j)) & 0xFu), s, bias);
}

extern "C" __global__ void gptq_unpack_u8(const uint32_t* __restrict__ qweight, uint8_t* __restrict__ q_out, int K,
                                          int N) {
    const int n = blockIdx.x * blockDim.x + threadIdx.x;
    const int kp = blockIdx.y;
    if (n >= N || kp >= K / 8) return;
    const uint32_t w = qweight[(size_t)kp * N + n];
#pragma unroll
    for (int j = 0; j < 8; ++j) q_out[((size_t)kp * 8 + j) * N + n] = (uint8_t)((w >> (4 * j)) & 0xFu);
}

// ---------------------------------------------------------------------------
// Dense bf16 [N,K] matrix times vector (LM head, in_proj_a/b): one warp per
// output row, 128-bit loads, fp32 accumulation in a fixed order.
// Replaces the reference's lm_head launch (src/launcher.s:2903-2970).
// ---------------------------------------------------------------------------
extern "C" __global__ void __launch_bounds__(256) dense_bf16_gemv(const __grid_constant__ lb_dense_params p) {
    extern __shared__ __align__(16) float xsm[]; // [K] fp32 + 40
    float* red = xsm + p.K;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    pdl_wait();
    if (p.x_mode == LB_X_F16) {
        const __half* xh = reinterpret_cast<const __half*>(p.x);
        for (int i = tid; i < p.K; i += blockDim.x) xsm[i] = __half2float(xh[i]);
    } else {
        const float* xf = reinterpret_cast<const float*>(p.x);
        float rinv = 1.f;
        if (p.x_mode == LB_X_F32_RMSNORM) {
            float ss = 0.f;
            for (int i = tid; i < p.K; i += blockDim.x) ss += xf[i] * xf[i];
            ss = block_sum(ss, red);
            rinv = rsqrtf(ss / (float)p.K + p.eps);
        }
        const uint16_t* nw = reinterpret_cast<const uint16_t*>(p.norm_w);
        for (int i = tid; i < p.K; i += blockDim.x) {
            float v = xf[i];
            if (p.x_mode == LB_X_F32_RMSNORM) v = v * rinv * (1.0f + bf16_bits_to_f32(nw[i]));
            xsm[i] = __half2float(__float2half_rn(v)); // activations are fp16 on this path
        }
    }
    __syncthreads();
    pdl_launch_dependents();
    const int nwarps = blockDim.x >> 5;
    for (int n = blockIdx.x * nwarps + warp; n < p.N; n += gridDim.x * nwarps) {
        const uint4* wr = reinterpret_cast<const uint4*>(p.w + (size_t)n * p.K);
        float a0 = 0.f, a1 = 0.f;
        for (int i = lane; i < p.K / 8; i += 32) {
            uint4 w = __ldcs(wr + i);
            const float4 xa = *reinterpret_cast<const float4*>(xsm + i * 8);
            const float4 xb = *reinterpret_cast<const float4*>(xsm + i * 8 + 4);
            a0 = fmaf(__uint_as_float(w.x << 16), xa.x, a0);
            a1 = fmaf(__uint_as_float(w.x & 0xffff0000u), xa.y, a1);
            a0 = fmaf(__uint_as_float(w.y << 16), xa.z, a0);
            a1 = fmaf(__uint_as_float(w.y & 0xffff0000u), xa.w, a1);
            a0 = fmaf(__uint_as_float(w.z << 16), xb.x, a0);
            a1 = fmaf(__uint_as_float(w.z & 0xffff0000u), xb.y, a1);
            a0 = fmaf(__uint_as_float(w.w << 16), xb.z, a0);
            a1 = fmaf(__uint_as_float(w.w & 0xffff0000u), xb.w, a1);
        }
        float t = warp_sum(a0 + a1);
        if (lane == 0) p.y[n] = t;
    }
}
