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
//   * Up to 32 tokens: products of a 5-bit integer and an fp16 value are exact in the fp32 accumulator; the
//     fp16 group scale multiplies the group's fp32 sum, so no weight is ever rounded.  33..64 tokens (one
//     warp keeps all 64 tokens' accumulators, so there is no room for per-group sums): the A registers are
//     (q - z) * s rounded to fp16, the dequantised weight the reference's own batched kernel multiplies
//     (kernels/projection_gemm.sass:477-631).
//   * The CTA is 8 warps = 8 column sets (128 columns).  Packed words
//     are prefetched three or four K-groups ahead in registers; the activations travel K-group by K-group through a
//     cp.async ring of as many stages in shared memory (16-byte chunks; rows of 320 bytes, so that the 128-bit
//     reads of a quarter-warp - two token rows x four chunks - cover all banks).
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
#define BG_XROW 320     // bytes per staged activation row: 256 + 64, so that odd rows start 16 banks further on
#define BG_PSTRIDE 132  // floats per row of the partial tile

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

struct bg_cursor { // where the lane's next K-group starts in the three weight buffers
    const uint32_t* q;
    const uint16_t* s;
    const uint32_t* z; // NULL: zero-point 8
    size_t N;
};

__device__ __forceinline__ void bg_load_group(bg_group& w, bg_cursor& c) {
#pragma unroll
    for (int j = 0; j < 4; ++j) w.w[j] = __ldg(reinterpret_cast<const uint2*>(c.q + (size_t)(4 * j) * c.N));
    w.s2 = __ldg(reinterpret_cast<const uint32_t*>(c.s));
    w.zw = c.z ? __ldg(c.z) : 0x88888888u;
    c.q += 16 * c.N;
    c.s += c.N;
    if (c.z) c.z += c.N / 8;
}

// byte I of a packed word (q0 | q1 << 4) as the fp16 pair (q0 - z, q1 - z)
template <int I>
__device__ __forceinline__ __half2 bg_pair(uint32_t w, __half2 mul, __half2 add) {
    const uint32_t v = __byte_perm(w, 0u, 0x4040u | I | (I << 8));
    return __hfma2(u32_as_h2(lop3_and_or(v, 0x00f0000fu, 0x64006400u)), mul, add);
}
// (-(1024 + z), -(64 + z)) as fp16 bits: 1024 + z = 0x6400 + z, 64 + z = 0x5400 + 16 z
__device__ __forceinline__ __half2 bg_bias(uint32_t z) { return u32_as_h2((0xE400u + z) | ((0xD400u + (z << 4)) << 16)); }

template <int NB, bool SCALED, int D> // a warp's NB blocks of 8 tokens; SCALED: A = (q - z) * s in fp16, no per-group sums;
                                      // D K-groups ahead: packed words in registers, activations in shared memory
__device__ __forceinline__ void gemm_int4_body(const lb_bgemm_params& p, unsigned char* smem) {
    constexpr int R = NB * 8, THREADS = BG_CSETS * 32;
    constexpr int CH = (R * 16 + THREADS - 1) / THREADS; // 16-byte activation chunks a thread copies per K-group
    unsigned char* xs = smem;                 // [D][R][BG_XROW]
    float* pt = reinterpret_cast<float*>(smem); // [R][BG_PSTRIDE], over the activation ring once the products are done
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int n0 = blockIdx.x * BG_COLS + warp * 16;
    const bool live = n0 < p.N; // N % 16 == 0
    const int groups = p.K / 128, KS = (int)gridDim.y;
    const int g_begin = (int)(((long long)blockIdx.y * groups) / KS), g_end = (int)(((long long)(blockIdx.y + 1) * groups) / KS);

    float acc[NB][4];
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) acc[nb][0] = acc[nb][1] = acc[nb][2] = acc[nb][3] = 0.f;

    // activations: thread copies chunk m (k = 8m..8m+7) of token rows b0, b0 + 16, ...
    const int b0 = tid >> 4, m = tid & 15;
    const uint16_t* xsrc = p.x + (size_t)g_begin * 128 + m * 8; // + b * K per row
    const uint32_t xdst = (uint32_t)(b0 * BG_XROW + m * 16);
    auto copy_x = [&](int grp, int stage) {
        if (grp < g_end) {
#pragma unroll
            for (int c = 0; c < CH; ++c) {
                const int b = b0 + c * 16;
                if (b < R) {
                    const bool valid = b < p.B;
                    cp_async16(xs + (size_t)stage * R * BG_XROW + xdst + c * 16 * BG_XROW, xsrc + (size_t)(valid ? b : 0) * p.K, valid);
                }
            }
            xsrc += 128;
        }
        cp_async_commit(); // one commit per K-group, empty or not: the wait below counts groups
    };

    bg_cursor cur_ptr;
    cur_ptr.N = (size_t)p.N;
    cur_ptr.q = p.qweight + ((size_t)g_begin * 16 + t) * p.N + n0 + 2 * g;
    cur_ptr.s = p.scales + (size_t)g_begin * p.N + n0 + 2 * g;
    cur_ptr.z = p.qzeros ? p.qzeros + (size_t)g_begin * (p.N / 8) + (n0 >> 3) + (g >> 2) : nullptr;
    bg_group ring[D];
#pragma unroll
    for (int u = 0; u < D; ++u)
        if (live && g_begin + u < g_end) bg_load_group(ring[u], cur_ptr);
#pragma unroll
    for (int s = 0; s < D - 1; ++s) copy_x(g_begin + s, s);

    const __half2 mul = u32_as_h2(0x2C003C00u); // (1, 1/16)
    const uint32_t xoff = (uint32_t)(g * BG_XROW + t * 16); // chunk 4j + t of row g: + 64 j
    for (int base = g_begin; base < g_end; base += D) {
#pragma unroll
        for (int u = 0; u < D; ++u) { // both rings have D entries: K-group base + u uses entry u of each
            const int grp = base + u;
            if (grp < g_end) { // uniform over the CTA
                cp_async_wait<D - 2>(); // this thread's chunks of K-group grp have landed
                __syncthreads();                // everybody's have, and everybody is done with K-group grp - 1
                copy_x(grp + D - 1, (u + D - 1) % D);
                const bg_group cur = ring[u];
                if (live && grp + D < g_end) bg_load_group(ring[u], cur_ptr);
                if (live) {
                    const uint32_t za = (cur.zw >> (8 * (g & 3))) & 0xFu, zb = (cur.zw >> (8 * (g & 3) + 4)) & 0xFu;
                    const __half2 addA = bg_bias(za), addB = bg_bias(zb);
                    const __half2 sA = __half2half2(__low2half(u32_as_h2(cur.s2))), sB = __half2half2(__high2half(u32_as_h2(cur.s2)));
                    float ga[SCALED ? 1 : NB][4];
                    if (!SCALED) {
#pragma unroll
                        for (int nb = 0; nb < NB; ++nb) ga[nb][0] = ga[nb][1] = ga[nb][2] = ga[nb][3] = 0.f;
                    }
                    const unsigned char* xrow = xs + (size_t)u * R * BG_XROW + xoff;
#pragma unroll
                    for (int j = 0; j < 4; ++j) { // packed row 4j + t: k = 8 (4j + t) .. + 7
                        const uint32_t wa = cur.w[j].x, wb = cur.w[j].y;
                        __half2 h[8] = {bg_pair<0>(wa, mul, addA), bg_pair<0>(wb, mul, addB), bg_pair<1>(wa, mul, addA), bg_pair<1>(wb, mul, addB),
                                        bg_pair<2>(wa, mul, addA), bg_pair<2>(wb, mul, addB), bg_pair<3>(wa, mul, addA), bg_pair<3>(wb, mul, addB)};
                        if (SCALED) {
#pragma unroll
                            for (int i = 0; i < 8; ++i) h[i] = __hmul2(h[i], (i & 1) ? sB : sA);
                        }
#pragma unroll
                        for (int nb = 0; nb < NB; ++nb) { // the 8 activations of token 8 nb + g this packed row multiplies
                            const uint4 xq = *reinterpret_cast<const uint4*>(xrow + nb * 8 * BG_XROW + 64 * j);
                            float(&d)[4] = SCALED ? acc[nb] : ga[SCALED ? 0 : nb];
                            mma_f16(d, h2_as_u32(h[0]), h2_as_u32(h[1]), h2_as_u32(h[2]), h2_as_u32(h[3]), xq.x, xq.y);
                            mma_f16(d, h2_as_u32(h[4]), h2_as_u32(h[5]), h2_as_u32(h[6]), h2_as_u32(h[7]), xq.z, xq.w);
                        }
                    }
                    if (!SCALED) {
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
    }
    cp_async_wait<0>();
    pdl_launch_dependents();
    __syncthreads(); // the partial tile goes where the activations were
    // partial tile: d0, d1 = column 2g, tokens 2t and 2t + 1; d2, d3 = column 2g + 1
#pragma unroll
    for (int nb = 0; nb < NB; ++nb)
#pragma unroll
        for (int i = 0; i < 4; ++i) pt[(nb * 8 + 2 * t + (i & 1)) * BG_PSTRIDE + warp * 16 + 2 * g + (i >> 1)] = acc[nb][i];
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

#define BG_KERNEL(name, NB, SCALED, D)                                                                                   \
    extern "C" __global__ void __launch_bounds__(256, 2) name(const __grid_constant__ lb_bgemm_params p) {             \
        extern __shared__ __align__(16) unsigned char bg_smem[];                                                       \
        pdl_wait();                                                                                                    \
        gemm_int4_body<NB, SCALED, D>(p, bg_smem);                                                                     \
    }
BG_KERNEL(gemm_int4_mma_b8, 1, false, 4)  // up to 8 tokens
BG_KERNEL(gemm_int4_mma_b16, 2, false, 4) // up to 16
BG_KERNEL(gemm_int4_mma_b32, 4, false, 3) // up to 32
BG_KERNEL(gemm_int4_mma_b64, 8, true, 3)  // up to 64
