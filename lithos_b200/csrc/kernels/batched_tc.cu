// Batched int4 projection on the 5th-generation tensor cores (tcgen05 + TMEM) for 9..128 tokens on sm_100a:
// Y[b][n] = sum_k W(k,n) X[b][k], W in the GPTQ buffers of the batch-1 GEMV (qweight [K/8,N], scales fp16
// [K/128,N], qzeros [K/128,N/8] or NULL = zero-point 8; inference/gemv.ls:44-130), X fp16 [B,K],
// Y fp32 or fp16 [B,N].  The reference's batched kernel is kernels/projection_gemm.sass:390-631
// (int4 -> fp16 into shared memory, then 16x8x16 tensor-core products); the product here is one
// tcgen05.mma of 128 weight columns x NT tokens x 16 k per instruction, accumulated in tensor memory.
//
// One CTA = 128 output columns x one K slice: 16 dequantising warps, one issuing thread, one activation thread.
// Per K-group (128 k):
//   * every dequantising thread converts 4 packed words of one column (prefetched four groups earlier): a packed
//     word is 8 consecutive k of one column, so its eight fp16 values (q - z) * s - q - z exact through the 0x6400
//     exponent trick, then one fp16 multiply: the weight the reference kernel multiplies - are one 16-byte
//     shared-memory store into the K-major operand tile with the 128-byte swizzle: two halves of 64 k, a row of
//     128 bytes per column, 16-byte slot (chunk % 8) ^ (column % 8) inside the row;
//   * the activations of the group arrive by two tiled TMA loads (64 k x NT tokens each, 128-byte swizzle by the
//     copy engine, tokens past the batch zero-filled), as many groups ahead as activation stages fit (3..16), in the
//     same layout with tokens as rows; warp 0 checks their arrival before it signs the stage as full;
//   * each warp fences its stores for the async proxy and arrives on the stage's "full" mbarrier; the issuing
//     thread waits for it, issues the eight tcgen05.mma (k = 16 each: the descriptor's
//     start address steps 32 bytes inside the swizzle atom) of the group and commits them to the "free" mbarriers
//     of the weight stage and of the activation stage, which the dequantising warps and the activation thread wait
//     for before they refill them.  No CTA-wide barrier inside the loop: the warps drift apart by up to four stages.
// (With unswizzled core-matrix tiles the same products took ~170 cycles each and bounded the loop together with
// the conversion; with the swizzled tiles 64 tokens cost what 16 do.)
// Epilogue: warps 0-3 read the accumulator (lane = column, TMEM column = token) with tcgen05.ld into the
// partial tile in shared memory; K slices (the CTAs of a cluster) are added in rank order through
// distributed shared memory exactly as in the mma.sync kernel of batched.cu.
// Every wait is bounded and reports through the status word; TMEM is freed on every path.
#include "common.cuh"
#include "params.h"

#define TC_COLS 128    // weight columns per CTA = M of the product
#define TC_DQ_THREADS 512                // dequantising threads (16 warps)
#define TC_WORDS (16 * TC_COLS / TC_DQ_THREADS) // packed words (of one column) a thread converts per K-group
#define TC_THREADS (TC_DQ_THREADS + 64)   // + one warp whose lane 0 issues the products + one whose lane 0 brings the activations
#define TC_STAGES 4
#define TC_RING 4 // K-groups of packed words a thread keeps in registers ahead of its conversion (a multiple of TC_STAGES)
#define TC_PSTRIDE 132                 // floats per row of the partial tile
#define TC_TMEM_COLS 128
#define TC_TA_COLS 512    // weights in tensor memory: accumulator in columns 0..255 (one per token), weight stage s in columns
#define TC_TA_A0 256      // 256 + 64 s .. + 63

__device__ __forceinline__ uint32_t tc_cluster_rank() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ void tc_cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ float tc_ld_cluster(const float* local_ptr, uint32_t rank) {
    uint32_t remote; float v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(local_ptr)), "r"(rank));
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
    return v;
}
// ---- tcgen05 ---------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* dst_smem, uint32_t cols) { // one full warp
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) { // the same warp
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
// shared-memory operand descriptor, K-major, 128-byte swizzle: start address, leading byte offset (unused by this
// layout) and stride byte offset (between groups of 8 rows) in 16-byte units, descriptor version 1 in bits 46-48
__device__ __forceinline__ uint64_t tc_smem_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)(lbo_bytes >> 4) << 16) | ((uint64_t)(sbo_bytes >> 4) << 32) | (1ull << 46) |
           (2ull << 61); // layout type 2: 128-byte swizzle
}
// instruction descriptor of kind::f16: fp32 accumulator, fp16 A and B, both K-major, N >> 3 at bit 17, M >> 4 at bit 24
__device__ __forceinline__ uint32_t tc_idesc(uint32_t M, uint32_t N) { return (1u << 4) | ((N >> 3) << 17) | ((M >> 4) << 24); }
__device__ __forceinline__ void tc_mma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
                 "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
                 : "memory");
}
__device__ __forceinline__ void tc_commit(uint64_t* bar) { // the barrier fires when every tcgen05.mma issued so far by this thread is done
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) { // 32 lanes x 16 consecutive columns
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
                   "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr)
                 : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
// 16 consecutive 32-bit columns of this thread's TMEM lane (the warp's lanes 32 (warp % 4) .. + 31), registers -> tensor memory
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint4& a, const uint4& b, const uint4& c, const uint4& d) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};" ::"r"(taddr), "r"(a.x),
                 "r"(a.y), "r"(a.z), "r"(a.w), "r"(b.x), "r"(b.y), "r"(b.z), "r"(b.w), "r"(c.x), "r"(c.y), "r"(c.z), "r"(c.w), "r"(d.x), "r"(d.y),
                 "r"(d.z), "r"(d.w)
                 : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// the product with the A operand in tensor memory (lane = row of A, a 32-bit column = two consecutive k)
__device__ __forceinline__ void tc_mma_ta(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d_tmem),
                 "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
                 : "memory");
}

__device__ __forceinline__ uint32_t tc_lop3_and_or(uint32_t a, uint32_t mask, uint32_t bits) { // (a & mask) | bits
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(a), "r"(mask), "r"(bits));
    return r;
}
__device__ __forceinline__ uint32_t tc_h2_bits(__half2 h) { return *reinterpret_cast<uint32_t*>(&h); }
__device__ __forceinline__ __half2 tc_bits_h2(uint32_t u) { return *reinterpret_cast<__half2*>(&u); }
// byte I of a packed word (q0 | q1 << 4) as the fp16 pair ((q0 - z) s, (q1 - z) s): (1024 + q0, 1024 + 16 q1) by
// mask-and-or, (q0 - z, q1 - z) by one fma with (1, 1/16) and (-(1024 + z), -(64 + z)), both exact, then the scale
template <int I>
__device__ __forceinline__ uint32_t tc_pair(uint32_t w, __half2 mul, __half2 add, __half2 s) {
    const uint32_t v = __byte_perm(w, 0u, 0x4040u | I | (I << 8));
    return tc_h2_bits(__hmul2(__hfma2(tc_bits_h2(tc_lop3_and_or(v, 0x00f0000fu, 0x64006400u)), mul, add), s));
}

// One tiled TMA load of 64 k of the activations of a K-group: box 64 k (128 bytes) x NT tokens of X [B, K], written with
// the 128-byte swizzle: the K-major operand tile with the tokens as rows.  Tokens past the batch are filled with zeros
// by the copy engine.
__device__ __forceinline__ void tc_tma_x(uint32_t dst_smem, const void* tmap, int k, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst_smem),
                 "l"(tmap), "r"(k), "r"(0), "r"(smem_u32(bar))
                 : "memory");
}

// Bounded wait of the single-thread roles and of each converting warp's lane 0 on a pipeline mbarrier: a tight loop of
// non-blocking test_wait (try_wait parks the thread and wakes it late; these waits sit on the critical path of every
// K-group), 16M polls at most, no global timer.
__device__ __forceinline__ bool tc_test_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok)
                 : "r"(smem_u32(bar)), "r"(parity)
                 : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool tc_wait(uint64_t* bar, uint32_t parity) {
    for (uint32_t i = 0; i < (1u << 24); ++i)
        if (tc_test_wait(bar, parity)) return true;
    return false;
}

struct tc_group { // a thread's share of one K-group: TC_WORDS consecutive packed rows (8 k each) of one column
    uint32_t w[TC_WORDS];
    uint32_t s;  // its fp16 scale (u16 load)
    uint32_t zw; // the zero-point word of its octet, as loaded (the nibble is taken out when the group is used)
};

#define TC_SBO 1024                    // bytes between groups of 8 rows: 8 rows of 128 bytes (one 128-byte swizzle atom)
#define TC_A_HALF (TC_COLS * 128)      // one 64-k half of the weight tile: 128 rows of 128 bytes
#define TC_A_STAGE (2 * TC_A_HALF)     // one K-group of dequantised weights: 32 KB
#define TC_X_STAGES 16                  // most activation stages (16 tokens); fewer for more tokens, see xstages
#define TC_FAIL_FREE 0x1101u           // status: a stage's products never completed
#define TC_FAIL_DONE 0x1102u           // status: the last products never completed
#define TC_FAIL_FULL 0x1103u           // status: a stage was never filled

// G: K-groups per hand-off between the converting warps and the issuing thread (1 or 2).
// TA: the dequantised weights go to TENSOR memory instead of shared memory (tcgen05.st; lane = weight column, a 32-bit
// column = two consecutive k: the A operand of tcgen05.mma read from tensor memory).  Per K-group that takes 32 KB of
// stores and 32 KB of operand reads off the shared-memory port and the swizzled stores and the proxy fence out of the
// converting warps; the activations get the whole shared memory (6 stages at 128 tokens), so two K-groups per hand-off
// fit at every token count.  4 - 8 % faster than the shared-memory operand tiles at every shape and token count measured.
template <int G, bool TA>
__device__ __forceinline__ void gemm_int4_tc_body(const lb_bgemm_params& p, unsigned char* tc_smem) {
    __shared__ __align__(8) uint64_t bar_free[TC_STAGES]; // a stage's products are done (tcgen05.commit)
    __shared__ __align__(8) uint64_t bar_full[TC_STAGES]; // a stage's weights are in place (one arrival per dequantising warp)
    __shared__ __align__(8) uint64_t bar_x[TC_X_STAGES];  // an activation stage has landed (TMA transaction bytes)
    __shared__ __align__(8) uint64_t bar_xfree[TC_X_STAGES]; // the products that read an activation stage are done
    __shared__ __align__(8) uint64_t bar_done;
    __shared__ uint32_t tmem_base_slot;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int NT = p.B > 128 ? 256 : p.B > 64 ? 128 : p.B > 32 ? 64 : p.B > 16 ? 32 : 16; // tokens the product carries (rows past B are zero)
    const int xstages = TA ? (NT > 128 ? 3 : NT > 64 ? 6 : NT > 32 ? 12 : TC_X_STAGES)
                           : (NT > 64 ? 3 : NT > 32 ? 5 : NT > 16 ? 10 : TC_X_STAGES); // activation stages that fit (beside the weight stages)
    const uint32_t x_stage_bytes = (uint32_t)NT * 256u, x_half = (uint32_t)NT * 128u; // a 64-k half: NT rows of 128 bytes
    unsigned char* a_smem = tc_smem;                          // [TC_STAGES][TC_A_STAGE]
    unsigned char* x_smem = tc_smem + (TA ? 0 : TC_STAGES * TC_A_STAGE); // [xstages][NT * 256]
    float* pt = reinterpret_cast<float*>(tc_smem);            // [NT][TC_PSTRIDE], over the weight stages once the products are done
    const int groups = p.K / 128, KS = (int)gridDim.y;
    const int g_begin = (int)(((long long)blockIdx.y * groups) / KS), g_end = (int)(((long long)(blockIdx.y + 1) * groups) / KS);

    if (tid == 0) {
        for (int s = 0; s < TC_STAGES; ++s) {
            mbar_init(&bar_free[s], 1);                    // (one per stage pair is used)
            mbar_init(&bar_full[s], TC_DQ_THREADS / 32);
        }
        for (int s = 0; s < TC_X_STAGES; ++s) {
            mbar_init(&bar_x[s], 1);
            mbar_init(&bar_xfree[s], 1);
        }
        mbar_init(&bar_done, 1);
        mbar_fence_init();
    }
    if (warp == 0) tmem_alloc(&tmem_base_slot, TA ? TC_TA_COLS : TC_TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_d = tmem_base_slot;
    pdl_wait();

    const uint32_t idesc = tc_idesc(TC_COLS, (uint32_t)NT);
    bool failed = false;
    if (warp < TC_DQ_THREADS / 32) {
        // ---------------- dequantising warps: fill stage after stage, never waiting for each other ----------------
        // weights: this thread's column and its four packed rows of every K-group
        const int nl = tid & (TC_COLS - 1), rq = tid >> 7; // column of the tile, which run of TC_WORDS packed rows (0..3)
        const int n = blockIdx.x * TC_COLS + nl;
        const bool live = n < p.N;
        const uint32_t* qptr = p.qweight + ((size_t)g_begin * 16 + TC_WORDS * rq) * p.N + n;
        const uint16_t* sptr = p.scales + (size_t)g_begin * p.N + n;
        const uint32_t* zptr = p.qzeros ? p.qzeros + (size_t)g_begin * (p.N / 8) + (n >> 3) : nullptr;
        const size_t row_stride = (size_t)p.N;
        auto load_group = [&](tc_group& w) {
#pragma unroll
            for (int j = 0; j < TC_WORDS; ++j) w.w[j] = __ldg(qptr + j * row_stride);
            w.s = __ldg(sptr);
            w.zw = zptr ? __ldg(zptr) : 0x88888888u;
            qptr += 16 * row_stride;
            sptr += row_stride;
            if (zptr) zptr += row_stride / 8;
        };
        tc_group ring[TC_RING]; // packed words of the next TC_RING K-groups
#pragma unroll
        for (int u = 0; u < TC_RING; ++u) {
#pragma unroll
            for (int j = 0; j < TC_WORDS; ++j) ring[u].w[j] = 0u;
            ring[u].s = 0u;
            ring[u].zw = 0x88888888u;
            if (live && g_begin + u < g_end) load_group(ring[u]);
        }
        const __half2 mul = tc_bits_h2(0x2C003C00u); // (1, 1/16)
        // chunk c (k = 8c..8c+7) of column nl: half c / 8, row nl, 16-byte slot (c % 8) ^ (nl % 8) of the row (128-byte swizzle)
        const uint32_t a_row = (uint32_t)(nl * 128), a_xor = (uint32_t)(nl & 7);
        const int zshift = 4 * (n & 7);
        // K-groups are handed over G at a time (G weight stages share one "full" and one "free" barrier): every hand-off is a
        // shared-memory round trip behind the stores, so fewer of them is what counts; G = 2 unless only three activation
        // stages fit (128 tokens), where a hand-off of two would leave the activation thread one stage to work ahead
        int pit = 0, xs_c = 0;
        uint32_t xs_ph = 0u;
        for (int base = g_begin; base < g_end && !failed; base += TC_RING) {
#pragma unroll
            for (int up = 0; up < TC_RING / G; ++up) { // TC_RING / G == TC_STAGES / G hand-off slots
                const int g0 = base + G * up;
                if (g0 < g_end && !failed) {
                    const int cnt = g_end - g0 < G ? g_end - g0 : G; // K-groups in this hand-off
                    uint4 v[G][TC_WORDS];
#pragma unroll
                    for (int h = 0; h < G; ++h) {
                        const tc_group cur = ring[G * up + h];
                        if (live && g0 + h + TC_RING < g_end) load_group(ring[G * up + h]);
                        const uint32_t z = (cur.zw >> zshift) & 0xFu;
                        const __half2 add = tc_bits_h2((0xE400u + z) | ((0xD400u + (z << 4)) << 16)); // (-(1024 + z), -(64 + z))
                        const __half2 sc = tc_bits_h2((cur.s & 0xFFFFu) * 0x10001u);
#pragma unroll
                        for (int j = 0; j < TC_WORDS; ++j) // a packed row = the 8 k of one core-matrix row
                            v[h][j] = make_uint4(tc_pair<0>(cur.w[j], mul, add, sc), tc_pair<1>(cur.w[j], mul, add, sc), tc_pair<2>(cur.w[j], mul, add, sc),
                                                 tc_pair<3>(cur.w[j], mul, add, sc));
                    }
                    // these stages held the K-groups four back: wait until their products are done
                    // (lane 0 polls for its warp; the vote orders the others behind it)
                    if (pit >= TC_STAGES / G && lane == 0 && !tc_wait(&bar_free[up], (uint32_t)((pit / (TC_STAGES / G) - 1) & 1))) {
                        failed = true;
                        if (p.status) atomicExch(p.status, TC_FAIL_FREE);
                    }
                    failed = __any_sync(0xffffffffu, failed); // the warp goes on, or leaves the loop, together
                    if (TA) {
                        static_assert(TC_WORDS == 4, "a thread's K-group share is 16 columns of tensor memory");
#pragma unroll
                        for (int h = 0; h < G; ++h)
                            if (h < cnt)
                                tmem_st16(tmem_d + ((uint32_t)(32 * (warp & 3)) << 16) + (uint32_t)(TC_TA_A0 + 64 * (G * up + h) + 16 * rq), v[h][0], v[h][1],
                                          v[h][2], v[h][3]);
                        tmem_st_wait();
                        tc_fence_before();
                    } else {
#pragma unroll
                        for (int h = 0; h < G; ++h) {
                            unsigned char* a_stage = a_smem + (G * up + h) * TC_A_STAGE + a_row;
#pragma unroll
                            for (int j = 0; j < TC_WORDS; ++j) {
                                const uint32_t c = (uint32_t)(TC_WORDS * rq + j);
                                if (h < cnt) *reinterpret_cast<uint4*>(a_stage + (c >> 3) * TC_A_HALF + (((c & 7) ^ a_xor) << 4)) = v[h][j];
                            }
                        }
                        fence_proxy_async_smem(); // generic-proxy stores before the tensor core reads them
                    }
                    __syncwarp();
                    if (lane == 0) {
                        // warp 0 also vouches for the activations of these K-groups, so that the issuing thread polls one barrier only
                        if (warp == 0) {
                            bool okx = tc_wait(&bar_x[xs_c], xs_ph);
                            if (cnt > 1) {
                                const int xn = xs_c + 1 == xstages ? 0 : xs_c + 1;
                                okx = okx && tc_wait(&bar_x[xn], xn == 0 ? xs_ph ^ 1u : xs_ph);
                            }
                            if (!okx && p.status) atomicExch(p.status, TC_FAIL_FULL);
                        }
                        mbar_arrive(&bar_full[up]);
                    }
                    for (int h = 0; h < cnt; ++h)
                        if (++xs_c == xstages) { xs_c = 0; xs_ph ^= 1u; }
                    ++pit;
                }
            }
        }
    } else if (warp == TC_DQ_THREADS / 32 && lane == 0) {
        // ---------------- issuing thread: eight products per K-group as soon as its weights and activations are in place ----------------
        const uint64_t a_desc0 = tc_smem_desc(smem_u32(a_smem), 16, TC_SBO), x_desc0 = tc_smem_desc(smem_u32(x_smem), 16, TC_SBO);
        int pit = 0, xstage = 0;
        for (int g0 = g_begin; g0 < g_end; g0 += G, ++pit) {
            const int up = pit % (TC_STAGES / G);
            const int cnt = g_end - g0 < G ? g_end - g0 : G;
            if (!tc_wait(&bar_full[up], (uint32_t)((pit / (TC_STAGES / G)) & 1))) { // weights stored, activations landed (warp 0 checked)
                failed = true;
                if (p.status) atomicExch(p.status, TC_FAIL_FULL);
                break;
            }
            tc_fence_after();
            for (int h = 0; h < cnt; ++h) {
                // descriptors: the start-address field counts 16-byte units
                const uint64_t a_desc = a_desc0 + (uint64_t)(((G * up + h) * TC_A_STAGE) >> 4), x_desc = x_desc0 + (uint64_t)((xstage * x_stage_bytes) >> 4);
#pragma unroll
                for (int kk = 0; kk < 8; ++kk) { // k = 16 kk .. + 15: two k chunks
                    const uint64_t xd = x_desc + (uint64_t)(((kk >> 2) * x_half + (kk & 3) * 32) >> 4);
                    const uint32_t acc = (pit > 0 || h > 0 || kk > 0) ? 1u : 0u;
                    if (TA) tc_mma_ta(tmem_d, tmem_d + (uint32_t)(TC_TA_A0 + 64 * (G * up + h) + 8 * kk), xd, idesc, acc);
                    else tc_mma(tmem_d, a_desc + (uint64_t)(((kk >> 2) * TC_A_HALF + (kk & 3) * 32) >> 4), xd, idesc, acc);
                }
                tc_commit(&bar_xfree[xstage]);
                xstage = xstage + 1 == xstages ? 0 : xstage + 1;
            }
            tc_commit(&bar_free[up]);
        }
        tc_commit(&bar_done); // fires when every product issued above is done
    } else if (warp == TC_DQ_THREADS / 32 + 1 && lane == 0) {
        // ---------------- activation thread: two tiled TMA loads per K-group, up to xstages groups ahead ----------------
        int j = 0, xs = 0;
        for (int grp = g_begin; grp < g_end; ++grp, ++j) {
            if (j >= xstages && !tc_wait(&bar_xfree[xs], (uint32_t)((j / xstages - 1) & 1))) {
                if (p.status) atomicExch(p.status, TC_FAIL_FREE);
                break; // the issuing thread then gives up on this stage's barrier and reports too
            }
            mbar_arrive_expect_tx(&bar_x[xs], x_stage_bytes);
            tc_tma_x(smem_u32(x_smem + (size_t)xs * x_stage_bytes), p.tmap_x, grp * 128, &bar_x[xs]);
            tc_tma_x(smem_u32(x_smem + (size_t)xs * x_stage_bytes + x_half), p.tmap_x, grp * 128 + 64, &bar_x[xs]);
            xs = xs + 1 == xstages ? 0 : xs + 1;
        }
    }
    pdl_launch_dependents();
    const bool done = mbar_wait(&bar_done, 0);
    if (!done && tid == 0 && p.status) atomicExch(p.status, TC_FAIL_DONE);
    tc_fence_after();
    failed = __syncthreads_or((failed || !done) ? 1 : 0) != 0;
    // accumulator -> partial tile: TMEM lane = column of the tile, TMEM column = token; warp w may touch lanes 32w..32w+31
    if (!failed && warp < 4) {
        for (int c = 0; c < NT / 16; ++c) {
            uint32_t r[16];
            tmem_ld16(tmem_d + ((uint32_t)(32 * warp) << 16) + (uint32_t)(c * 16), r);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 16; ++j) pt[(c * 16 + j) * TC_PSTRIDE + 32 * warp + lane] = __uint_as_float(r[j]);
        }
    }
    tc_fence_before();
    tc_cluster_sync(); // every CTA of the cluster has its tile in place (a plain CTA barrier when there is no cluster)
    const uint32_t rank = KS > 1 ? tc_cluster_rank() : 0u;
    const int cols = min(TC_COLS, p.N - (int)blockIdx.x * TC_COLS);
    if (!failed) {
        for (int i = tid; i < NT * TC_COLS; i += TC_THREADS) {
            const int b = i / TC_COLS, c = i % TC_COLS;
            if (b >= p.B || c >= cols || (b % KS) != (int)rank) continue;
            float v = 0.f;
            if (KS == 1) v = pt[b * TC_PSTRIDE + c];
            else
                for (int q = 0; q < KS; ++q) v += tc_ld_cluster(pt + b * TC_PSTRIDE + c, (uint32_t)q);
            const size_t o = (size_t)b * p.N + (size_t)blockIdx.x * TC_COLS + c;
            if (p.y_f32) reinterpret_cast<float*>(p.y)[o] = v;
            else reinterpret_cast<__half*>(p.y)[o] = __float2half_rn(v);
        }
    }
    if (KS > 1) tc_cluster_sync(); // nobody leaves while a neighbour still reads its tile
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem_d, TA ? TC_TA_COLS : TC_TMEM_COLS);
}

extern "C" __global__ void __launch_bounds__(TC_THREADS, 1) gemm_int4_tc(const __grid_constant__ lb_bgemm_params p) { // up to 64 tokens
    extern __shared__ __align__(1024) unsigned char tc_smem[];
    gemm_int4_tc_body<2, false>(p, tc_smem);
}
extern "C" __global__ void __launch_bounds__(TC_THREADS, 1) gemm_int4_tc_g1(const __grid_constant__ lb_bgemm_params p) { // 65..128 tokens
    extern __shared__ __align__(1024) unsigned char tc_smem[];
    gemm_int4_tc_body<1, false>(p, tc_smem);
}
extern "C" __global__ void __launch_bounds__(TC_THREADS, 1) gemm_int4_tc_ta(const __grid_constant__ lb_bgemm_params p) { // weights through tensor memory
    extern __shared__ __align__(1024) unsigned char tc_smem[];
    gemm_int4_tc_body<2, true>(p, tc_smem);
}
// 129..256 tokens: one product of 128 x 256 x 16 per k step (the weights of a K-group are converted once for twice the tokens);
// three activation stages of 64 KB fit, so K-groups are handed over one at a time
extern "C" __global__ void __launch_bounds__(TC_THREADS, 1) gemm_int4_tc_ta_g1(const __grid_constant__ lb_bgemm_params p) {
    extern __shared__ __align__(1024) unsigned char tc_smem[];
    gemm_int4_tc_body<1, true>(p, tc_smem);
}
