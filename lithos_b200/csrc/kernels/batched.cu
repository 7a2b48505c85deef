// Batched int4 projection for up to 64 tokens at once on sm_100a: Y[b][n] = sum_k W(k,n) X[b][k] with the
// GPTQ operands of the batch-1 GEMV (qweight [K/8,N], scales fp16 [K/128,N], qzeros [K/128,N/8] or NULL
// = zero-point 8; inference/gemv.ls:44-130) and fp16 activations X [B,K], fp32 (or fp16) results [B,N].
//
// The weights are read ONCE for the whole batch: the batch is the N dimension of a tensor-core product
// (mma.sync.m16n8k16, fp16 operands, fp32 accumulation; weight columns are the M rows).
//   * A warp owns 16 output columns and up to 32 tokens.  The order of the k index inside a product is
//     free as long as both operands agree, so it is chosen for the weight side: lane (g, t) owns, for the
//     column pair (2g, 2g+1), the packed rows t, t+4, t+8, t+12 of a K-group - four 64-bit loads, every
//     byte of every 32-byte sector used - and a k-step takes its A registers out of one packed word: a
//     byte (q0 | q1 << 4) copied into both halves of a register, masked with 0x00f0000f and or-ed with
//     0x64006400, is the fp16 pair (1024 + q0, 1024 + 16 q1); one fma with (1, 1/16) and
//     (-(1024 + z), -(64 + z)) turns it into the exact integers (q0 - z, q1 - z).  The lane's B registers
//     of two k-steps are one 128-bit read of the 8 activations that packed word multiplies.
//   * Products of a 5-bit integer and an fp16 value are exact in the fp32 accumulator; the fp16 group scale
//     multiplies the group's fp32 sum, so no weight is ever rounded.
//   * The CTA is 8 column sets (128 columns) x 1 or 2 token halves (256 or 512 threads).  Packed words
//     are prefetched four K-groups ahead in registers; the activations travel K-group by K-group through a
//     four-stage cp.async ring in shared memory (16-byte chunks, chunk index xor-ed with 4 (row & 1) so
//     that the 128-bit reads of a quarter-warp cover all banks).
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
#define BG_STAGES 4     // K-groups of activations in the shared-memory ring
#define BG_PSTRIDE 132  // floats per row of the partial tile
#define BG_DEPTH 4      // K-groups of packed words in registers ahead of the products

__device__ __forceinline__ void mma_f16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
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
__device__ __forceinline__ uint32_t lop3_and_or(uint32_t a, uint32_t mask, uint32_t bits) { // (a & mask) | bits
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(a), "r"(mask), "r"(bits));
    return r;
}
__device__ __forceinline__ uint32_t h2_as_u32(__half2 h) { return *reinterpret_cast<uint32_t*>(&h); }
__device__ __forceinline__ __half2 u32_as_h2(uint32_t u) { return *reinterpret_cast<__half2*>(&u); }

__device__ __forceinline__ void cp_async16(void* dst_smem, const void* src, bool valid) { // zero fill when !valid
    const uint32_t n = valid ? 16u : 0u;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(dst_smem)), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

struct bg_group { // lane (g, t): packed rows t, t+4, t+8, t+12 of columns n0 + 2g (.x) and n0 + 2g + 1 (.y) of one K-group
    uint2 w[4];
    uint32_t s2; // the two fp16 scales
    uint32_t zw; // the zero-point word of the lane's octet (0x88888888 without qzeros)
};

__device__ __forceinline__ void bg_load_group(bg_group& w, const lb_bgemm_params& p, int grp, int n0, int g, int t) {
    const uint32_t* q = p.qweight + ((size_t)grp * 16 + t) * p.N + n0 + 2 * g;
#pragma unroll
    for (int j = 0; j < 4; ++j) w.w[j] = __ldg(reinterpret_cast<const uint2*>(q + (size_t)(4 * j) * p.N));
    w.s2 = __ldg(reinterpret_cast<const uint32_t*>(p.scales + (size_t)grp * p.N + n0 + 2 * g));
    w.zw = p.qzeros ? __ldg(p.qzeros + (size_t)grp * (p.N / 8) + (n0 >> 3) + (g >> 2)) : 0x88888888u;
}

// byte I of a packed word (q0 | q1 << 4) as the fp16 pair (q0 - z, q1 - z)
template <int I>
__device__ __forceinline__ uint32_t bg_pair(uint32_t w, __half2 mul, __half2 add) {
    const uint32_t v = __byte_perm(w, 0u, 0x4040u | I | (I << 8));
    return h2_as_u32(__hfma2(u32_as_h2(lop3_and_or(v, 0x00f0000fu, 0x64006400u)), mul, add));
}

template <int NB, int TH> // a warp's NB blocks of 8 tokens; TH token halves per CTA
__device__ __forceinline__ void gemm_int4_body(const lb_bgemm_params& p, unsigned char* smem) {
    constexpr int R = NB * 8 * TH, THREADS = BG_CSETS * 32 * TH;
    constexpr int CH = (R * 16 + THREADS - 1) / THREADS; // 16-byte activation chunks a thread copies per K-group
    unsigned char* xs = smem;                                                        // [BG_STAGES][R][256 B]
    float* pt = reinterpret_cast<float*>(smem + (size_t)BG_STAGES * R * 256);        // [R][BG_PSTRIDE]
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int cs = warp % BG_CSETS, tb = (warp / BG_CSETS) * NB * 8; // column set, first token
    const int n0 = blockIdx.x * BG_COLS + cs * 16;
    const bool live = n0 < p.N; // N % 16 == 0
    const int groups = p.K / 128, KS = (int)gridDim.y;
    const int g_begin = (int)(((long long)blockIdx.y * groups) / KS), g_end = (int)(((long long)(blockIdx.y + 1) * groups) / KS);

    float acc[NB][4];
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) acc[nb][0] = acc[nb][1] = acc[nb][2] = acc[nb][3] = 0.f;

    // chunk m (k = 8m..8m+7) of token row b of a K-group sits at chunk position m ^ 4 (b & 1) of the row
    auto copy_x = [&](int grp, int stage) {
        if (grp < g_end) {
#pragma unroll
            for (int c = 0; c < CH; ++c) {
                const int i = tid + c * THREADS, b = i >> 4, m = i & 15;
                if (i < R * 16) {
                    const bool valid = b < p.B;
                    cp_async16(xs + ((size_t)stage * R + b) * 256 + ((m ^ ((b & 1) << 2)) << 4),
                               p.x + (size_t)(valid ? b : 0) * p.K + (size_t)grp * 128 + m * 8, valid);
                }
            }
        }
        cp_async_commit(); // one commit per K-group, empty or not: the wait below counts groups
    };

    bg_group ring[BG_DEPTH];
#pragma unroll
    for (int u = 0; u < BG_DEPTH; ++u)
        if (live && g_begin + u < g_end) bg_load_group(ring[u], p, g_begin + u, n0, g, t);
#pragma unroll
    for (int s = 0; s < BG_STAGES - 1; ++s) copy_x(g_begin + s, s);

    const __half2 mul = u32_as_h2(0x2C003C00u); // (1, 1/16)
    for (int base = g_begin; base < g_end; base += BG_DEPTH) {
#pragma unroll
        for (int u = 0; u < BG_DEPTH; ++u) { // BG_DEPTH == BG_STAGES: stage of K-group base + u is u
            const int grp = base + u;
            if (grp < g_end) { // uniform over the CTA
                cp_async_wait<BG_STAGES - 2>(); // this thread's chunks of K-group grp have landed
                __syncthreads();                // everybody's have, and everybody is done with K-group grp - 1
                copy_x(grp + BG_STAGES - 1, (u + BG_STAGES - 1) % BG_STAGES);
                const bg_group cur = ring[u];
                if (live && grp + BG_DEPTH < g_end) bg_load_group(ring[u], p, grp + BG_DEPTH, n0, g, t);
                if (live) {
                    const uint32_t za = (cur.zw >> (8 * (g & 3))) & 0xFu, zb = (cur.zw >> (8 * (g & 3) + 4)) & 0xFu;
                    // q0 - z = (1024 + q0) - (1024 + z),  q1 - z = (1024 + 16 q1) / 16 - (64 + z): exact in fp16
                    const __half2 addA = __halves2half2(__ushort_as_half((unsigned short)(0xE400u + za)), __int2half_rn(-64 - (int)za));
                    const __half2 addB = __halves2half2(__ushort_as_half((unsigned short)(0xE400u + zb)), __int2half_rn(-64 - (int)zb));
                    float ga[NB][4];
#pragma unroll
                    for (int nb = 0; nb < NB; ++nb) ga[nb][0] = ga[nb][1] = ga[nb][2] = ga[nb][3] = 0.f;
                    const unsigned char* xrow = xs + ((size_t)u * R + tb + g) * 256;
#pragma unroll
                    for (int j = 0; j < 4; ++j) { // packed row 4j + t: k = 8 (4j + t) .. + 7
                        const uint32_t wa = cur.w[j].x, wb = cur.w[j].y;
                        const uint32_t a0 = bg_pair<0>(wa, mul, addA), a1 = bg_pair<0>(wb, mul, addB);
                        const uint32_t a2 = bg_pair<1>(wa, mul, addA), a3 = bg_pair<1>(wb, mul, addB);
                        const uint32_t c0 = bg_pair<2>(wa, mul, addA), c1 = bg_pair<2>(wb, mul, addB);
                        const uint32_t c2 = bg_pair<3>(wa, mul, addA), c3 = bg_pair<3>(wb, mul, addB);
#pragma unroll
                        for (int nb = 0; nb < NB; ++nb) { // the 8 activations of token tb + 8 nb + g this packed row multiplies
                            const uint4 xq = *reinterpret_cast<const uint4*>(xrow + (size_t)nb * 8 * 256 + (((4 * j + t) ^ ((g & 1) << 2)) << 4));
                            mma_f16(ga[nb], a0, a1, a2, a3, xq.x, xq.y);
                            mma_f16(ga[nb], c0, c1, c2, c3, xq.z, xq.w);
                        }
                    }
                    const float2 sc = __half22float2(u32_as_h2(cur.s2));
#pragma unroll
                    for (int nb = 0; nb < NB; ++nb) {
                        acc[nb][0] = fmaf(sc.x, ga[nb][0], acc[nb][0]); acc[nb][1] = fmaf(sc.x, ga[nb][1], acc[nb][1]);
                        acc[nb][2] = fmaf(sc.y, ga[nb][2], acc[nb][2]); acc[nb][3] = fmaf(sc.y, ga[nb][3], acc[nb][3]);
                    }
                }
            }
        }
    }
    cp_async_wait<0>();
    pdl_launch_dependents();
    // partial tile: d0, d1 = column 2g, tokens 2t and 2t + 1; d2, d3 = column 2g + 1
#pragma unroll
    for (int nb = 0; nb < NB; ++nb)
#pragma unroll
        for (int i = 0; i < 4; ++i) pt[(tb + nb * 8 + 2 * t + (i & 1)) * BG_PSTRIDE + cs * 16 + 2 * g + (i >> 1)] = acc[nb][i];
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

static_assert(BG_DEPTH == BG_STAGES, "the K-group loop indexes both rings with the same unrolled counter");

#define BG_KERNEL(name, NB, TH)                                                                                        \
    extern "C" __global__ void __launch_bounds__(256 * TH, 2 / TH) name(const __grid_constant__ lb_bgemm_params p) {           \
        extern __shared__ __align__(16) unsigned char bg_smem[];                                                       \
        pdl_wait();                                                                                                    \
        gemm_int4_body<NB, TH>(p, bg_smem);                                                                            \
    }
BG_KERNEL(gemm_int4_mma_b8, 1, 1)  // up to 8 tokens
BG_KERNEL(gemm_int4_mma_b16, 2, 1) // up to 16
BG_KERNEL(gemm_int4_mma_b32, 4, 1) // up to 32
BG_KERNEL(gemm_int4_mma_b64, 4, 2) // up to 64: two warps per column set with 32 tokens each
