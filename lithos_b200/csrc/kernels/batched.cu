// Batched int4 projection for up to 64 tokens at once on sm_100a: Y[b][n] = sum_k W(k,n) X[b][k] with the
// GPTQ operands of the batch-1 GEMV (qweight [K/8,N], scales fp16 [K/128,N], qzeros [K/128,N/8] or NULL
// = zero-point 8; inference/gemv.ls:44-130) and fp16 activations X [B,K], fp32 (or fp16) results [B,N].
//
// The weights are read ONCE for the whole batch: the batch is the N dimension of a tensor-core product.
//   * A warp owns 16 output columns and up to 32 tokens.  Per 16 k it turns its packed words into an fp16
//     A fragment in registers - the integers q - z, exact in fp16 (the 0x6400 exponent trick: one mask,
//     one or, one subtract per pair) - and issues one mma.sync.m16n8k16 per 8 tokens against the
//     activations staged in shared memory.  Products of a 5-bit integer and an fp16 value are exact in the
//     fp32 accumulator; the fp16 group scale multiplies the group's fp32 sum, so no weight is ever rounded.
//   * The CTA is 8 column sets (128 columns) x 1 or 2 token halves (256 or 512 threads) and stages one
//     K-group (128 k) of all tokens at a time, double buffered; the next group's packed words are already
//     in registers while the current group is multiplied.
//   * Narrow matrices are split along K over the CTAs of a thread-block cluster (grid.y = cluster.y <= 8):
//     every CTA leaves its partial tile in shared memory and the ranks add them in rank order through
//     distributed shared memory, each rank the token rows b = rank (mod cluster size): a fixed order, so
//     the result does not depend on timing.
// This is the legacy tensor path (mma.sync): it serves batch 2..64 until a tcgen05 skinny GEMM (weights
// dequantised to shared memory, accumulators in TMEM) replaces it for batch >= 16.
#include "common.cuh"
#include "params.h"

#define BG_CSETS 8      // column sets of 16 columns per CTA
#define BG_COLS 128     // columns per CTA
#define BG_XSTRIDE 136  // halves per staged activation row: 128 + 8, so that the 8 rows of a fragment hit different banks
#define BG_PSTRIDE 132  // floats per row of the partial tile

__device__ __forceinline__ void mma_f16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// nibbles 2t and 2t+1 of a packed word as the fp16 pair (q0 - z, q1 - z); zbias = (1024 + z, 1024 + z)
__device__ __forceinline__ uint32_t nibble_pair(uint32_t w, int t, __half2 zbias) {
    const uint32_t v = w >> (8 * t);
    const uint32_t bits = (v & 0xFu) | ((v & 0xF0u) << 12) | 0x64006400u; // (1024 + q0, 1024 + q1) as fp16
    const __half2 h = __hsub2(*reinterpret_cast<const __half2*>(&bits), zbias);
    return *reinterpret_cast<const uint32_t*>(&h);
}

__device__ __forceinline__ uint32_t bg_cluster_rank() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ void bg_cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ float bg_ld_cluster(const float* local_ptr, uint32_t rank) {
    uint32_t remote; float v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(local_ptr)), "r"(rank));
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
    return v;
}

struct bg_group { // one K-group of a warp's 16 columns, as loaded
    uint32_t wa[16], wb[16]; // packed rows of columns n0 + g and n0 + 8 + g
    uint16_t sa, sb;         // their fp16 scales
    uint32_t za, zb;         // their zero-points
};

__device__ __forceinline__ void bg_load_group(bg_group& w, const lb_bgemm_params& p, int grp, int n0, int g) {
    const uint32_t* q = p.qweight + (size_t)grp * 16 * p.N + n0 + g;
#pragma unroll
    for (int r = 0; r < 16; ++r) {
        w.wa[r] = __ldg(q + (size_t)r * p.N);
        w.wb[r] = __ldg(q + (size_t)r * p.N + 8);
    }
    w.sa = __ldg(p.scales + (size_t)grp * p.N + n0 + g);
    w.sb = __ldg(p.scales + (size_t)grp * p.N + n0 + 8 + g);
    w.za = w.zb = 8u;
    if (p.qzeros) { // 16 columns = two zero-point words
        w.za = (__ldg(p.qzeros + (size_t)grp * (p.N / 8) + (n0 >> 3)) >> (4 * g)) & 0xFu;
        w.zb = (__ldg(p.qzeros + (size_t)grp * (p.N / 8) + (n0 >> 3) + 1) >> (4 * g)) & 0xFu;
    }
}

template <int NB, int TH> // a warp's NB blocks of 8 tokens; TH token halves per CTA
__device__ __forceinline__ void gemm_int4_body(const lb_bgemm_params& p, unsigned char* smem) {
    constexpr int R = NB * 8 * TH, THREADS = BG_CSETS * 32 * TH;
    __half* xs = reinterpret_cast<__half*>(smem);                                         // [2][R][BG_XSTRIDE]
    float* pt = reinterpret_cast<float*>(smem + (size_t)2 * R * BG_XSTRIDE * sizeof(__half)); // [R][BG_PSTRIDE]
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int cs = warp % BG_CSETS, tb = (warp / BG_CSETS) * NB * 8; // column set, first token
    const int n0 = blockIdx.x * BG_COLS + cs * 16;
    const bool live = n0 < p.N; // N % 16 == 0
    const int groups = p.K / 128, KS = (int)gridDim.y;
    const int g_begin = (int)(((long long)blockIdx.y * groups) / KS), g_end = (int)(((long long)(blockIdx.y + 1) * groups) / KS);

    float acc[NB][4];
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) acc[nb][0] = acc[nb][1] = acc[nb][2] = acc[nb][3] = 0.f;

    auto stage_x = [&](int grp, int buf) { // all tokens' 128 activations of one K-group, 16 B per thread and step
        __half* dst = xs + (size_t)buf * R * BG_XSTRIDE;
        for (int i = tid; i < R * 16; i += THREADS) {
            const int b = i >> 4, c16 = i & 15;
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            if (b < p.B) v = __ldg(reinterpret_cast<const uint4*>(p.x + (size_t)b * p.K + (size_t)grp * 128) + c16);
            *reinterpret_cast<uint4*>(dst + b * BG_XSTRIDE + c16 * 8) = v;
        }
    };

    bg_group nxt;
    if (g_begin < g_end) {
        if (live) bg_load_group(nxt, p, g_begin, n0, g);
        stage_x(g_begin, 0);
    }
    __syncthreads();
    for (int grp = g_begin; grp < g_end; ++grp) {
        const int buf = (grp - g_begin) & 1;
        bg_group cur = nxt;
        if (grp + 1 < g_end) {
            if (live) bg_load_group(nxt, p, grp + 1, n0, g);
            stage_x(grp + 1, buf ^ 1);
        }
        if (live) {
            const __half2 zba = __half2half2(__ushort_as_half((unsigned short)(0x6400u + cur.za)));
            const __half2 zbb = __half2half2(__ushort_as_half((unsigned short)(0x6400u + cur.zb)));
            float ga[NB][4];
#pragma unroll
            for (int nb = 0; nb < NB; ++nb) ga[nb][0] = ga[nb][1] = ga[nb][2] = ga[nb][3] = 0.f;
            const __half* xb = xs + (size_t)buf * R * BG_XSTRIDE + (tb + g) * BG_XSTRIDE + 2 * t;
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) { // 16 k per step = packed rows 2 ks and 2 ks + 1
                // A (16 columns x 16 k): a0 = (column g, k 2t..), a1 = (column g + 8, k 2t..), a2, a3 = the same at k + 8
                const uint32_t a0 = nibble_pair(cur.wa[2 * ks], t, zba), a1 = nibble_pair(cur.wb[2 * ks], t, zbb);
                const uint32_t a2 = nibble_pair(cur.wa[2 * ks + 1], t, zba), a3 = nibble_pair(cur.wb[2 * ks + 1], t, zbb);
#pragma unroll
                for (int nb = 0; nb < NB; ++nb) { // B (16 k x 8 tokens): b0 = (k 2t.., token g), b1 = the same at k + 8
                    const __half* xr = xb + nb * 8 * BG_XSTRIDE + ks * 16;
                    mma_f16(ga[nb], a0, a1, a2, a3, *reinterpret_cast<const uint32_t*>(xr), *reinterpret_cast<const uint32_t*>(xr + 8));
                }
            }
            const float sa = __half2float(__ushort_as_half(cur.sa)), sb = __half2float(__ushort_as_half(cur.sb));
#pragma unroll
            for (int nb = 0; nb < NB; ++nb) {
                acc[nb][0] = fmaf(sa, ga[nb][0], acc[nb][0]); acc[nb][1] = fmaf(sa, ga[nb][1], acc[nb][1]);
                acc[nb][2] = fmaf(sb, ga[nb][2], acc[nb][2]); acc[nb][3] = fmaf(sb, ga[nb][3], acc[nb][3]);
            }
        }
        __syncthreads(); // the next group's activations are in place; this group's buffer is free for the one after
    }
    pdl_launch_dependents();
    // partial tile: d0, d1 = column g, tokens 2t and 2t + 1; d2, d3 = column g + 8
#pragma unroll
    for (int nb = 0; nb < NB; ++nb)
#pragma unroll
        for (int i = 0; i < 4; ++i) pt[(tb + nb * 8 + 2 * t + (i & 1)) * BG_PSTRIDE + cs * 16 + g + (i >> 1) * 8] = acc[nb][i];
    bg_cluster_sync(); // every CTA of the cluster has its tile in place (a plain CTA barrier when there is no cluster)
    const uint32_t rank = KS > 1 ? bg_cluster_rank() : 0u;
    const int cols = min(BG_COLS, p.N - (int)blockIdx.x * BG_COLS);
    for (int i = tid; i < R * BG_COLS; i += THREADS) {
        const int b = i / BG_COLS, c = i % BG_COLS;
        if (b >= p.B || c >= cols || (b % KS) != (int)rank) continue;
        float v = 0.f;
        if (KS == 1) v = pt[b * BG_PSTRIDE + c];
        else
            for (int q = 0; q < KS; ++q) v += bg_ld_cluster(pt + b * BG_PSTRIDE + c, (uint32_t)q);
        const size_t o = (size_t)b * p.N + (size_t)blockIdx.x * BG_COLS + c;
        if (p.y_f32) reinterpret_cast<float*>(p.y)[o] = v;
        else reinterpret_cast<__half*>(p.y)[o] = __float2half_rn(v);
    }
    if (KS > 1) bg_cluster_sync(); // nobody leaves while a neighbour still reads its tile
}

// up to 32 tokens: 256 threads, every warp takes all tokens
extern "C" __global__ void __launch_bounds__(256) gemm_int4_mma(const __grid_constant__ lb_bgemm_params p) {
    extern __shared__ __align__(16) unsigned char bg_smem[];
    pdl_wait();
    const int nb = (p.B + 7) / 8;
    if (nb <= 1) gemm_int4_body<1, 1>(p, bg_smem);
    else if (nb == 2) gemm_int4_body<2, 1>(p, bg_smem);
    else gemm_int4_body<4, 1>(p, bg_smem);
}

// 33..64 tokens: 512 threads, two warps per column set with 32 tokens each
extern "C" __global__ void __launch_bounds__(512) gemm_int4_mma_wide(const __grid_constant__ lb_bgemm_params p) {
    extern __shared__ __align__(16) unsigned char bg_smem[];
    pdl_wait();
    gemm_int4_body<4, 2>(p, bg_smem);
}
