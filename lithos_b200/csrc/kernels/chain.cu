// The persistent kernel of the decode step on sm_100a: a chain of GPTQ int4 GEMVs, DeltaNet mixers and (under
// tensor parallelism) all-reduces in ONE launch of one CTA per SM, with a grid barrier between entries.
//
// The decode step of the reference runs its projections as separate launches
// (src/launcher.s:1226-1535, one launch_gemv per projection; the mixer as ten more, :832-844); at batch 1
// each projection moves 25-90 MB and a B200 drains that in 4-14 us, so launch gaps, pipeline fill and the
// split-K tail of every launch cost as much as the streaming itself.  Here everything between two attention
// kernels is one launch:
//   * CTA c owns whole columns of every GEMV (a strip of octets, all of K), so its results are
//     final: no partial sums, counters or atomics between CTAs, and the sum order is fixed.
//   * The weights come from a strip-packed copy (gemv_pack_strips below; layout in params.h) in
//     which a CTA's strip is one contiguous byte range, cut into stages of 4 K-groups x 16
//     columns (4352 bytes).  Whenever one of a warp's ring slots is free the warp takes the next stage of the
//     CTA's list that nobody has asked for (a counter in shared memory), requests it with a plain 1-D bulk
//     copy into that slot, waits for it on the slot's mbarrier and consumes it alone.  No producer warp, no
//     block-wide synchronisation inside a GEMV, and the 16 warps finish a GEMV together however unevenly the
//     stages arrive.  Weights are constants, so the requests run on into the NEXT GEMV of the chain while
//     the block finishes the current one: the rings of all SMs keep HBM busy across entry boundaries.
//   * A stage item is (K-group, pair of octets): two 128-bit loads per lane give the packed words, which go
//     into the tensor core as they are (a byte = two nibbles) and once more with the low nibbles masked off;
//     four m16n8k32 u8 x s8 steps against the activation digit planes give the exact integer dot products
//     of 16 columns (ch_item below); scale and zero-point are applied in fp32 per group.  A stage leaves its
//     16 column sums in the stage's own slot, and the slots of a column are added in the order of K: the
//     result does not depend on which warp took which stage.
//   * A DeltaNet entry runs the mixer of a layer ((value head, 32-column slab) units, four teams of 128
//     threads per CTA of which two compute the gate dot products for the other two; deltanet_core.cuh).
//     Under tensor parallelism a row-parallel GEMV exchanges its partial sums with the other GPUs in its own
//     epilogue (8-byte (value, generation) words stored into every rank's buffer; comm_core.cuh).  The weight
//     rings stay full meanwhile.
//   * Between entries the block meets the other blocks at a grid barrier (an arrival counter in
//     global memory: release-add, acquire poll, bounded spin).  All CTAs are resident: the grid is one
//     CTA per SM and a CTA takes more than half of an SM's shared memory.
//   * Where a GEMV's input vector is the result of the GEMV right before it (out projection -> gate/up -> down -> next
//     input projection), no grid barrier separates them.  The producer's threads store every result a second time as
//     an 8-byte word (value, tag) into the entry's mailbox -- one store, delivered whole -- with tag = launch base +
//     entry index; the consumer's activation-table loads read those words and simply repeat a row until all its tags
//     are this launch's.  The wait for the slowest producer and the table's trip to L2 become one, and the arrive /
//     poll / release-fence round trips of a barrier disappear.  A buffer is never overwritten while someone may still
//     read it: a CTA reaches the epilogue of entry o+1 only after it has seen every CTA's results of entry o, which a
//     CTA publishes after it has finished reading entry o-1's.
// Activations written inside the launch are read through L2 only (ld.global.cg / ld.volatile).
#include "gemv_core.cuh"
#include "deltanet_core.cuh"
#include "comm_core.cuh"

#define CH_W LB_CHAIN_WARPS
#define CH_GC LB_CHAIN_GC
#define CH_SYNC() __syncthreads()
#define CH_NO_STAGE 0xffffffffu // slot descriptor: nothing was asked for (the list is exhausted)

// timeline stamps: the "memory" clobber keeps the read where it is written (between the block barriers and memory accesses around it)
__device__ __forceinline__ unsigned long long ch_clock() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%clock64;" : "=l"(t)::"memory");
    return t;
}
__device__ __forceinline__ unsigned long long ch_globaltimer() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)::"memory");
    return t;
}
__device__ __forceinline__ unsigned ld_acquire_gpu(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
// first octet of CTA c's strip
__device__ __forceinline__ int ch_start(int c, int units, int upo, int G) { return (int)((long long)c * units / G) * upo; }

struct __align__(16) ch_shared {
    float vals[LB_CHAIN_MAX_OCTETS * 8];
    float scratch[64];
    int op_n0[LB_CHAIN_MAX_OPS];     // first octet of this CTA's strip, per GEMV
    int op_no[LB_CHAIN_MAX_OPS];     // octets in the strip
    int op_np[LB_CHAIN_MAX_OPS];     // pairs in the strip (a trailing single octet counts as one)
    int op_nch[LB_CHAIN_MAX_OPS];    // chunks of CH_GC K-groups per pair
    int op_pre[LB_CHAIN_MAX_OPS + 1]; // stages of this CTA before each GEMV (prefix sums of op_np * op_nch)
    const unsigned char* op_packed[LB_CHAIN_MAX_OPS]; // the GEMV's strip-packed weights (a copy of the parameter, for indexed reads)
    uint32_t next; // next stage of the CTA's list that nobody has asked for yet
    uint32_t bad;  // a bounded wait ran out (set by any thread at any time)
    uint32_t snap; // copy of bad taken by thread 0 before a block barrier: the value all threads act on together
    float dn_ab[2][2]; // DeltaNet entry: the gate dot products (a, b) of the units of teams 0 and 1, from teams 2 and 3
    unsigned long long stamp[8]; // timeline stamps of the current entry (thread 0), copied out when the entry ends: a global store
                                 // in the middle of an entry would hold up the loads and stores behind it
};

// position in the CTA's stage list: GEMV o, pair of that GEMV's strip, chunk of CH_GC K-groups of the pair
struct ch_cursor {
    int o, pair, chunk;
};

struct ch_stage {
    const unsigned char* src;
    uint32_t bytes;
    int g0, gcount, recb;
};

__device__ __forceinline__ ch_stage ch_decode(const lb_chain_params& p, const ch_shared& sh, const ch_cursor& k) {
    const lb_chain_op& op = p.op[k.o];
    ch_stage s;
    s.recb = 2 * k.pair + 1 < sh.op_no[k.o] ? 2 * LB_CHAIN_RECORD : LB_CHAIN_RECORD; // a trailing single octet has half records
    s.g0 = k.chunk * CH_GC;
    s.gcount = min(CH_GC, op.kg - s.g0);
    s.src = op.packed + ((size_t)sh.op_n0[k.o] * op.kg + (size_t)k.pair * op.kg * 2) * LB_CHAIN_RECORD + (size_t)s.g0 * s.recb;
    s.bytes = (uint32_t)(s.gcount * s.recb);
    return s;
}

// D(16x8, s32) += A(16x32, u8) * B(32x8, s8); not volatile: a pure function of its operands, free to be scheduled
__device__ __forceinline__ void imma_nv(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// ---- the activation table (B operand) ------------------------------------------------------------------------------
// One block of CH_XG bytes per K-group.  A packed weight word holds 8 consecutive k as nibbles: byte i = (k = 2i in the
// low nibble, k = 2i + 1 in the high one).  The tensor-core step takes the word AS IT IS (byte = low + 16 high) against
// the digits of the even k, and the word with the low nibbles masked off (byte = 16 high) against the digits of the odd
// k and, in the neighbouring output column, of the even k again; low . even = first - third, high . odd = second / 16.
// So the int4 -> operand conversion is ONE logic instruction per 8 weights, and the block holds
//   [0, 192)    even-k digits: [plane 0..2][t 0..3][packed row t, t+4, t+8, t+12 of the group] as 4-byte words
//   [192, 384)  odd-k digits, same order
//   [384, 400)  float {16 * sum of the group's integers, 0, 0, 0}: what fragment lane t multiplies the zero-point with
// (CH_XG = 448 keeps both the 16-byte fragment loads and the prologue's 4-byte stores free of bank conflicts).
#define CH_XG LB_CHAIN_GROUP_BYTES
#define CH_X_ODD 192
#define CH_X_SUM 384

// per-lane constants of the stage loop
struct ch_lane {
    uint32_t w_off;   // this lane's 16 bytes inside a record
    uint32_t s_off;   // this lane's (scale, zero-point) inside a record
    uint32_t x1, x2;  // B-operand loads inside a group block: first (even-k digits of plane g/2), second (odd-k digits for even
                      // g, even-k digits for odd g); columns 6 and 7 of the product are never read, they repeat plane 2
    uint32_t xs;      // this lane's word of the group-sum entry
    float mul;        // 256^t / 16 for t < 3 (fragment lane t holds digit plane t), 0 for t = 3
};
__device__ __forceinline__ ch_lane ch_lane_make(int lane) {
    const int g = lane >> 2, t = lane & 3, pl = min(g >> 1, 2);
    ch_lane L;
    L.w_off = (uint32_t)lane * 16u;
    L.s_off = 512u + 4u * (uint32_t)g;
    L.x1 = (uint32_t)(pl * 64 + t * 16);
    L.x2 = (g & 1) ? L.x1 : CH_X_ODD + L.x1;
    L.xs = CH_X_SUM + 4u * (uint32_t)t;
    L.mul = t == 0 ? 0.0625f : t == 1 ? 16.0f : t == 2 ? 4096.0f : 0.0f;
    return L;
}

// One item: K-group (packed words wa, wb and (scale, zero-point) words sa, sb of this lane; table block `xg`) x pair of
// octets = 16 columns x 128 k as exact integer dot products.  Fragment rows 0-7 are the columns of the first octet, rows
// 8-15 those of the second (FULL = false: a single octet, wb = sb = 0).
// acc += scale * (16 * (w . digits of plane t) - zero * 16 * sum X [t = 0]) for this lane's column and digit plane.
template <bool FULL>
__device__ __forceinline__ void ch_item(const uint4& wa, const uint4& wb, uint32_t sa_bits, uint32_t sb_bits, const unsigned char* xg,
                                        const ch_lane& L, float& acc_a, float& acc_b) {
    const uint32_t H = 0xf0f0f0f0u;
    const uint4 b1 = *reinterpret_cast<const uint4*>(xg + L.x1);
    const uint4 b2 = *reinterpret_cast<const uint4*>(xg + L.x2);
    int d1[4] = {0, 0, 0, 0}, d2[4] = {0, 0, 0, 0};
    imma_nv(d1, wa.x, wb.x, wa.y, wb.y, b1.x, b1.y);
    imma_nv(d2, wa.x & H, wb.x & H, wa.y & H, wb.y & H, b2.x, b2.y);
    imma_nv(d1, wa.z, wb.z, wa.w, wb.w, b1.z, b1.w);
    imma_nv(d2, wa.z & H, wb.z & H, wa.w & H, wb.w & H, b2.z, b2.w);
    const float xs = *reinterpret_cast<const float*>(xg + L.xs);
    const float2 sa = __half22float2(*reinterpret_cast<const __half2*>(&sa_bits));
    acc_a = fmaf(sa.x, fmaf(-sa.y, xs, (float)(16 * (d1[0] - d2[1]) + d2[0])), acc_a);
    if (FULL) {
        const float2 sb = __half22float2(*reinterpret_cast<const __half2*>(&sb_bits));
        acc_b = fmaf(sb.x, fmaf(-sb.y, xs, (float)(16 * (d1[2] - d2[3]) + d2[2])), acc_b);
    }
}

// A whole stage (CH_GC items) in registers: the ring slot is read in one go, handed back to the copy engine, and the
// tensor-core work runs from registers and the activation table while the slot's next stage is already on its way.
template <bool FULL>
struct ch_stage_regs {
    uint4 wa[CH_GC], wb[CH_GC];
    uint32_t sa[CH_GC], sb[CH_GC];
    __device__ __forceinline__ void load(const unsigned char* stage, const ch_lane& L) {
        constexpr int RECB = FULL ? 2 * LB_CHAIN_RECORD : LB_CHAIN_RECORD;
#pragma unroll
        for (int j = 0; j < CH_GC; ++j) {
            const unsigned char* rec = stage + j * RECB;
            wa[j] = *reinterpret_cast<const uint4*>(rec + L.w_off);
            sa[j] = *reinterpret_cast<const uint32_t*>(rec + L.s_off);
            wb[j] = FULL ? *reinterpret_cast<const uint4*>(rec + LB_CHAIN_RECORD + L.w_off) : make_uint4(0u, 0u, 0u, 0u);
            sb[j] = FULL ? *reinterpret_cast<const uint32_t*>(rec + LB_CHAIN_RECORD + L.s_off) : 0u;
        }
    }
    __device__ __forceinline__ void compute(const unsigned char* xg, const ch_lane& L, float& acc_a, float& acc_b) const {
#pragma unroll
        for (int j = 0; j < CH_GC; ++j) ch_item<FULL>(wa[j], wb[j], sa[j], sb[j], xg + j * CH_XG, L, acc_a, acc_b);
    }
};

// A short stage (the tail of K: fewer than CH_GC items), straight from the ring slot.
template <bool FULL>
__device__ __forceinline__ void ch_stage_tail(const unsigned char* stage, const unsigned char* xg, int gcount, const ch_lane& L,
                                              float& acc_a, float& acc_b) {
    constexpr int RECB = FULL ? 2 * LB_CHAIN_RECORD : LB_CHAIN_RECORD;
#pragma unroll 1
    for (int j = 0; j < gcount; ++j) {
        const unsigned char* rec = stage + j * RECB;
        const uint4 wa = *reinterpret_cast<const uint4*>(rec + L.w_off);
        const uint4 wb = FULL ? *reinterpret_cast<const uint4*>(rec + LB_CHAIN_RECORD + L.w_off) : make_uint4(0u, 0u, 0u, 0u);
        const uint32_t sa = *reinterpret_cast<const uint32_t*>(rec + L.s_off);
        const uint32_t sb = FULL ? *reinterpret_cast<const uint32_t*>(rec + LB_CHAIN_RECORD + L.s_off) : 0u;
        ch_item<FULL>(wa, wb, sa, sb, xg + j * CH_XG, L, acc_a, acc_b);
    }
}

// silu of the 8 gate values of packed row r (zeros past the end of the vector)
__device__ __noinline__ void ch_gate_rows(const lb_chain_op& op, int r, int rows, float (&g)[8]) {
    float4 a = make_float4(0.f, 0.f, 0.f, 0.f), b = a;
    if (r < rows) {
        const float4* zv = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(op.aux1) + r * 8);
        a = __ldcg(zv);
        b = __ldcg(zv + 1);
    }
    g[0] = siluf_dev(a.x); g[1] = siluf_dev(a.y); g[2] = siluf_dev(a.z); g[3] = siluf_dev(a.w);
    g[4] = siluf_dev(b.x); g[5] = siluf_dev(b.y); g[6] = siluf_dev(b.z); g[7] = siluf_dev(b.w);
}

// The activation vector of one GEMV as exact integers, for the whole block: X_k = rint(x_k * 2^shift) with
// |X| < 2^22, split into three signed base-256 digits that become the B operand of the integer MMA (digit table
// layout: digit_row_word).  x_k is the fp16 activation (after the optional norm prologue), so X_k is EXACT for every
// element within 2^-11 of the vector maximum and off by at most max|x| * 2^-23 below that.  Returns 2^-shift.
// Thread tid owns packed rows tid, tid + 512, ... (NI of them at most); all global loads are issued before the
// first use, so the prologue costs one trip to L2, not one per row.
template <int NI>
__device__ __forceinline__ float ch_prologue(const lb_chain_op& op, ch_shared& sh, unsigned char* xtab, int tid, bool write_x,
                                             const unsigned long long* mailbox, uint32_t tag, uint32_t* status, unsigned long long* tl,
                                             const float (&gz)[2][8]) {
    const int lane = tid & 31, warp = tid >> 5;
    const int rows = op.K / 8;
    // a warp's rows of round i are 32 consecutive ones: when none of them exists the whole warp skips the round's arithmetic
#define CH_WARP_ROWS(i) ((tid & ~31) + (i) * LB_CHAIN_THREADS < rows)
    float pre_max = -1.f; // >= 0: the largest |h| is already known (no second block-wide exchange)
    uint32_t hv[NI][4]; // the row as 8 fp16 values
    if (op.x_mode == LB_X_F16) {
#pragma unroll
        for (int i = 0; i < NI; ++i) {
            const int r = tid + i * LB_CHAIN_THREADS;
            uint4 raw = make_uint4(0u, 0u, 0u, 0u);
            if (r < rows && !mailbox) raw = __ldcg(reinterpret_cast<const uint4*>(reinterpret_cast<const __half*>(op.x) + r * 8));
            hv[i][0] = raw.x; hv[i][1] = raw.y; hv[i][2] = raw.z; hv[i][3] = raw.w;
        }
        if (mailbox) { // the producer's (two fp16 values, tag) words: a row of 8 values is 4 words; repeat until all are this launch's
            const uint64_t t0 = globaltimer_ns(), limit = 2 * lb_wait_limit_ns(status); // twice: whoever the producers wait for reports first
            for (unsigned it = 0;; ++it) {
                bool ok = true;
#pragma unroll
                for (int i = 0; i < NI; ++i) {
                    const int r = tid + i * LB_CHAIN_THREADS;
                    if (r >= rows) continue;
                    const uint4 a = ld_volatile_v4(mailbox + (size_t)r * 4), b = ld_volatile_v4(mailbox + (size_t)r * 4 + 2);
                    ok = ok && a.y == tag && a.w == tag && b.y == tag && b.w == tag;
                    hv[i][0] = a.x; hv[i][1] = a.z; hv[i][2] = b.x; hv[i][3] = b.z;
                }
                if (ok) break;
                if ((it & 15u) == 15u && (it >= LB_WAIT_SPINS || globaltimer_ns() - t0 > limit || *reinterpret_cast<volatile uint32_t*>(status) != 0u)) {
                    atomicCAS(status, 0u, LB_DEV_TIMEOUT_COUNTER);
                    sh.bad = 1;
                    break;
                }
            }
        }
        if (tl && tid == 0) sh.stamp[3] = ch_clock(); // this thread's part of the input vector has arrived (mailbox) or been asked for
    } else {
        // the norm weights do not depend on the input vector: asked for before the wait for it
        uint4 wr[NI];
        if (op.x_mode == LB_X_F32_RMSNORM) {
#pragma unroll
            for (int i = 0; i < NI; ++i) {
                const int r = tid + i * LB_CHAIN_THREADS;
                wr[i] = r < rows ? __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(op.aux0) + r * 8)) : make_uint4(0u, 0u, 0u, 0u);
            }
        }
        float v[NI][8];
#pragma unroll
        for (int i = 0; i < NI; ++i) {
            const int r = tid + i * LB_CHAIN_THREADS;
            float4 a = make_float4(0.f, 0.f, 0.f, 0.f), b = a;
            if (r < rows && !mailbox) {
                const float4* xv = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(op.x) + r * 8);
                a = __ldcg(xv);
                b = __ldcg(xv + 1);
            }
            v[i][0] = a.x; v[i][1] = a.y; v[i][2] = a.z; v[i][3] = a.w;
            v[i][4] = b.x; v[i][5] = b.y; v[i][6] = b.z; v[i][7] = b.w;
        }
        if (mailbox) { // the producer's (fp32 value, tag) words: a row of 8 values is 8 words
            const uint64_t t0 = globaltimer_ns(), limit = 2 * lb_wait_limit_ns(status); // twice: whoever the producers wait for reports first
            for (unsigned it = 0;; ++it) {
                bool ok = true;
#pragma unroll
                for (int i = 0; i < NI; ++i) {
                    const int r = tid + i * LB_CHAIN_THREADS;
                    if (r >= rows) continue;
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const uint4 a = ld_volatile_v4(mailbox + (size_t)r * 8 + 2 * j);
                        ok = ok && a.y == tag && a.w == tag;
                        v[i][2 * j] = __uint_as_float(a.x);
                        v[i][2 * j + 1] = __uint_as_float(a.z);
                    }
                }
                if (ok) break;
                if ((it & 15u) == 15u && (it >= LB_WAIT_SPINS || globaltimer_ns() - t0 > limit || *reinterpret_cast<volatile uint32_t*>(status) != 0u)) {
                    atomicCAS(status, 0u, LB_DEV_TIMEOUT_COUNTER);
                    sh.bad = 1;
                    break;
                }
            }
        }
        if (tl && tid == 0) sh.stamp[3] = ch_clock();
        if (op.x_mode == LB_X_F32_RMSNORM) {
            // h = (x * (1 + w)) * rsqrt(mean x^2 + eps): the rows held by the block's threads are the whole vector.  The
            // product with (1 + w) comes first, so that the sum of squares and the largest |x (1 + w)| go through ONE
            // block-wide exchange: rounding is monotonic, so the largest |h| is the largest |x (1 + w)| times the factor.
            float ss = 0.f, um = 0.f;
#pragma unroll
            for (int i = 0; i < NI; ++i) {
                if (!CH_WARP_ROWS(i)) continue;
                const uint32_t ww[4] = {wr[i].x, wr[i].y, wr[i].z, wr[i].w};
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const float wf = __uint_as_float(j & 1 ? ww[j >> 1] & 0xffff0000u : ww[j >> 1] << 16);
                    ss += v[i][j] * v[i][j];
                    v[i][j] = v[i][j] * (1.0f + wf);
                    um = fmaxf(um, fabsf(v[i][j]));
                }
            }
            ss = warp_sum(ss);
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) um = fmaxf(um, __shfl_xor_sync(0xffffffffu, um, o));
            if (lane == 0) { sh.scratch[warp] = ss; sh.scratch[32 + warp] = um; }
            CH_SYNC();
            float tot = 0.f;
            um = 0.f;
#pragma unroll
            for (int w = 0; w < CH_W; ++w) { tot += sh.scratch[w]; um = fmaxf(um, sh.scratch[32 + w]); }
            const float rinv = rsqrtf(tot / (float)op.K + op.eps);
#pragma unroll
            for (int i = 0; i < NI; ++i)
#pragma unroll
                for (int j = 0; j < 8; ++j) v[i][j] *= rinv;
            pre_max = __half2float(__float2half_rn(um * rinv)); // the largest |h| after the fp16 rounding below
        } else if (NI <= 2 && op.x_mode == LB_X_F32_HEADNORM_SILU) { // (the host refuses this prologue for K > 8192: it would not fit the registers)
            // one head = 128 values = the 16 rows held by a 16-lane segment; h = x * rsqrt(mean_head x^2 + eps) * w * silu(z)
            const float4* wv = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(op.aux0) + (tid & 15) * 8);
            const float4 wa = __ldg(wv), wb = __ldg(wv + 1);
            const float hw[8] = {wa.x, wa.y, wa.z, wa.w, wb.x, wb.y, wb.z, wb.w};
            // silu(z) of this thread's rows: taken by the caller before the entry's barrier (op.early_gate), else here
            float z[NI][8];
#pragma unroll
            for (int i = 0; i < NI; ++i) {
                if (op.early_gate) {
#pragma unroll
                    for (int j = 0; j < 8; ++j) z[i][j] = gz[i][j];
                } else ch_gate_rows(op, tid + i * LB_CHAIN_THREADS, rows, z[i]);
            }
#pragma unroll
            for (int i = 0; i < NI; ++i) {
                float ss = 0.f;
#pragma unroll
                for (int j = 0; j < 8; ++j) ss += v[i][j] * v[i][j];
#pragma unroll
                for (int o = 8; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
                const float hr = rsqrtf(ss * (1.0f / 128.0f) + op.eps);
#pragma unroll
                for (int j = 0; j < 8; ++j) v[i][j] = v[i][j] * hr * hw[j] * z[i][j];
            }
        }
#pragma unroll
        for (int i = 0; i < NI; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const __half2 h = __floats2half2_rn(v[i][2 * j], v[i][2 * j + 1]);
                hv[i][j] = *reinterpret_cast<const uint32_t*>(&h);
            }
    }
    // the scale: max|x| * 2^shift in [2^21, 2^22); all-zero or non-finite vectors use shift 0
    float vmax = pre_max;
    if (pre_max < 0.f) {
        vmax = 0.f;
#pragma unroll
        for (int i = 0; i < NI; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&hv[i][j]));
                vmax = fmaxf(vmax, fmaxf(fabsf(f.x), fabsf(f.y)));
            }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) vmax = fmaxf(vmax, __shfl_xor_sync(0xffffffffu, vmax, o));
        if (lane == 0) sh.scratch[32 + warp] = vmax;
        CH_SYNC();
        vmax = 0.f;
#pragma unroll
        for (int w = 0; w < CH_W; ++w) vmax = fmaxf(vmax, sh.scratch[32 + w]);
    }
    int shift = 0;
    if (vmax > 0.f && vmax < 3.0e38f) shift = 21 - (int)((__float_as_uint(vmax) >> 23) & 0xffu) + 127;
    const float qscale = __uint_as_float((uint32_t)(127 + shift) << 23);
#pragma unroll
    for (int i = 0; i < NI; ++i) {
        if (!CH_WARP_ROWS(i)) continue;
        const int r = tid + i * LB_CHAIN_THREADS;
        const bool live = r < rows;
        // X = rint(x * 2^shift) = d0 + 256 d1 + 65536 d2 with every d in [-128, 127].  Y = X + 0x808080 has the unsigned bytes
        // d + 128, and the byte with its top bit flipped is d in two's complement.  Adding 1.5 * 2^23 in fp32 rounds x * 2^shift
        // to the nearest integer (ties to even) and leaves it in the low mantissa bits, so Y is one FMA and one integer add.
        uint32_t Y[8];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&hv[i][j]));
            Y[2 * j] = __float_as_uint(fmaf(f.x, qscale, 12582912.0f)) + (0x00808080u - 0x4B400000u);
            Y[2 * j + 1] = __float_as_uint(fmaf(f.y, qscale, 12582912.0f)) + (0x00808080u - 0x4B400000u);
        }
        uint32_t rs = ((Y[0] + Y[1]) + (Y[2] + Y[3])) + ((Y[4] + Y[5]) + (Y[6] + Y[7])); // 128 values below 2^24: no overflow
        // byte p of Y[0], Y[2], Y[4], Y[6] -> ev[p]; of Y[1], Y[3], Y[5], Y[7] -> od[p]
        uint32_t ev[3], od[3];
        {
            const uint32_t a = __byte_perm(Y[0], Y[2], 0x5140), b = __byte_perm(Y[4], Y[6], 0x5140);
            ev[0] = __byte_perm(a, b, 0x5410);
            ev[1] = __byte_perm(a, b, 0x7632);
            ev[2] = __byte_perm(__byte_perm(Y[0], Y[2], 0x0062), __byte_perm(Y[4], Y[6], 0x0062), 0x5410);
            const uint32_t c = __byte_perm(Y[1], Y[3], 0x5140), d = __byte_perm(Y[5], Y[7], 0x5140);
            od[0] = __byte_perm(c, d, 0x5410);
            od[1] = __byte_perm(c, d, 0x7632);
            od[2] = __byte_perm(__byte_perm(Y[1], Y[3], 0x0062), __byte_perm(Y[5], Y[7], 0x0062), 0x5410);
        }
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) rs += __shfl_xor_sync(0xffffffffu, rs, o); // the group's 16 rows
        if (live) {
            // packed row r of group r / 16: word (r & 15) >> 2 of fragment lane t = r & 3
            unsigned char* blk = xtab + (size_t)(r >> 4) * CH_XG + (r & 3) * 16 + ((r & 15) >> 2) * 4;
#pragma unroll
            for (int d = 0; d < 3; ++d) {
                *reinterpret_cast<uint32_t*>(blk + d * 64) = ev[d] ^ 0x80808080u;
                *reinterpret_cast<uint32_t*>(blk + CH_X_ODD + d * 64) = od[d] ^ 0x80808080u;
            }
            if ((lane & 15) == 0) // sum of X = sum of Y - 128 * 0x808080
                *reinterpret_cast<float4*>(xtab + (size_t)(r >> 4) * CH_XG + CH_X_SUM) =
                    make_float4(16.0f * (float)(int)(rs - 128u * 0x00808080u), 0.f, 0.f, 0.f);
            if (op.x_out && write_x) // every CTA holds the whole vector: one of them writes it out
                *reinterpret_cast<uint4*>(op.x_out + r * 8) = make_uint4(hv[i][0], hv[i][1], hv[i][2], hv[i][3]);
        }
    }
    CH_SYNC();
    return __uint_as_float((uint32_t)(127 - shift) << 23);
#undef CH_WARP_ROWS
}

extern "C" __global__ void __launch_bounds__(LB_CHAIN_THREADS, 1) gemv_chain(const __grid_constant__ lb_chain_params p) {
    extern __shared__ __align__(16) unsigned char smem[];
    __shared__ ch_shared sh;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int c = blockIdx.x, G = gridDim.x;
    const int NS = p.slots; // ring slots of every warp

    // shared memory: [ring: CH_W * NS stages][activation table][per-stage column sums][mbarriers][slot descriptors][stage list]
    unsigned char* xtab = smem + (size_t)CH_W * NS * LB_CHAIN_STAGE_BYTES;
    float* red = reinterpret_cast<float*>(xtab + (size_t)(p.table_rows / LB_GEMV_ROWS) * CH_XG + 64); // [red_slots][16]
    uint64_t* full = reinterpret_cast<uint64_t*>(red + (size_t)p.red_slots * 16);          // [CH_W * NS]
    uint32_t* slot_desc = reinterpret_cast<uint32_t*>(full + CH_W * NS);                   // [CH_W * NS]
    uint2* tab = reinterpret_cast<uint2*>(slot_desc + ((CH_W * NS + 1) & ~1));             // [tab_len]

    if (tid < CH_W * NS) mbar_init(&full[tid], 1);
    if (tid < p.n_ops) {
        const lb_chain_op& op = p.op[tid];
        const bool gemv = op.type == LB_CHAIN_OP_GEMV;
        const int n0 = gemv ? ch_start(c, op.units, op.upo, G) : 0, no = gemv ? ch_start(c + 1, op.units, op.upo, G) - n0 : 0;
        sh.op_n0[tid] = n0;
        sh.op_no[tid] = no;
        sh.op_np[tid] = (no + 1) / 2;
        sh.op_nch[tid] = (op.kg + CH_GC - 1) / CH_GC;
        sh.op_packed[tid] = op.packed;
    }
    if (tid == 0) {
        sh.bad = 0;
        sh.snap = 0;
        sh.next = 0;
    }
    mbar_fence_init();
    __syncthreads();
    if (tid == 0) {
        int acc = 0;
        for (int o = 0; o < p.n_ops; ++o) {
            sh.op_pre[o] = acc;
            acc += sh.op_np[o] * sh.op_nch[o];
        }
        sh.op_pre[p.n_ops] = acc;
    }
    __syncthreads();


    // ---- the CTA's stage list: all GEMVs of the chain in order, each pair-major in chunks of CH_GC K-groups, written down
    //      once as (offset, descriptor) words.  A warp takes the next stage nobody has asked for whenever one of its ring
    //      slots is free (a counter in shared memory), so the warps of a block finish a GEMV together however unevenly the
    //      stages arrive; what a stage adds to the column sums goes to the stage's own slot, so the result does not depend
    //      on who took what. ----
    const uint32_t total = min((uint32_t)sh.op_pre[p.n_ops], (uint32_t)p.tab_len);
    for (uint32_t k = tid; k < total; k += LB_CHAIN_THREADS) {
        int o = 0;
        while ((int)k >= sh.op_pre[o + 1]) ++o; // k < total, so this stops inside the list
        ch_cursor cur;
        cur.o = o;
        const int li = (int)k - sh.op_pre[o];
        cur.pair = li / sh.op_nch[o];
        cur.chunk = li - cur.pair * sh.op_nch[o];
        const ch_stage st = ch_decode(p, sh, cur);
        const uint32_t full_pair = st.recb == 2 * LB_CHAIN_RECORD;
        tab[k] = make_uint2((uint32_t)((st.src - p.op[o].packed) >> 4),
                            (uint32_t)o | ((uint32_t)cur.pair << 5) | ((uint32_t)st.g0 << 10) | ((uint32_t)st.gcount << 22) | (full_pair << 25));
    }
    __syncthreads();
    const uint64_t pol = l2_policy_evict_first();
    uint32_t req_slot = 0, use_slot = 0, use_par = 0; // the warp's ring: next slot to fill, next to consume and its mbarrier phase
    unsigned char* const ring = smem + (size_t)warp * NS * LB_CHAIN_STAGE_BYTES;
    uint64_t* const wfull = full + warp * NS;
    uint32_t* const wdesc = slot_desc + warp * NS; // per slot: the descriptor of the stage asked for, CH_NO_STAGE when none
    // Asking for a stage is lane 0's business alone (the other lanes learn about it from the slot's descriptor after the
    // next __syncwarp).  The index of the stage to ask for next is taken one request ahead: the shared-memory atomic has
    // long returned when the slot it is for becomes free.
    uint32_t next_k = 0;
    if (lane == 0) next_k = atomicAdd(&sh.next, 1u);
    auto request = [&]() { // weights never change: requests may run ahead of everything, the first ones start before griddepcontrol.wait
        if (lane == 0) {
            uint32_t d = CH_NO_STAGE;
            if (next_k < total) {
                const uint2 e = tab[next_k];
                const uint32_t bytes = ((e.y >> 22) & 7u) * ((e.y >> 25) & 1u ? 2u * LB_CHAIN_RECORD : (uint32_t)LB_CHAIN_RECORD);
                d = e.y;
                mbar_arrive_expect_tx(&wfull[req_slot], bytes);
                bulk_g2s(ring + (size_t)req_slot * LB_CHAIN_STAGE_BYTES, sh.op_packed[e.y & 31u] + ((size_t)e.x << 4), bytes, &wfull[req_slot], pol);
                next_k = atomicAdd(&sh.next, 1u);
            }
            wdesc[req_slot] = d;
        }
        req_slot = req_slot + 1 == (uint32_t)NS ? 0u : req_slot + 1;
    };
    for (int i = 0; i < NS; ++i) request();
    __syncwarp();

    const int fg = lane >> 2, ft = lane & 3;
    const ch_lane L = ch_lane_make(lane);
    pdl_wait(); // activations and barrier words belong to the stream order
    // tensor parallel: the exchange generation of this GPU, read once (every exchange of the launch counts up from it)
    unsigned ar_gen0 = 0, n_barriers = 0; // n_barriers: grid barriers passed (thread 0 only)
    int ar_done = 0;
    const lb_tp_params* ar_tp = nullptr;
    for (int o = 0; o < p.n_ops; ++o)
        if (p.op[o].type == LB_CHAIN_OP_GEMV && p.op[o].y_mode == LB_Y_TP_ALLREDUCE) {
            ar_tp = reinterpret_cast<const lb_tp_params*>(p.op[o].ext);
            break;
        }
    if (ar_tp) ar_gen0 = ar_tp->gen[0];
    const uint32_t tag_base = *reinterpret_cast<volatile uint32_t*>(p.sync + 2); // every CTA reads it before the last one out advances it
    for (int o = 0; o < p.n_ops; ++o) {
        const lb_chain_op& op = p.op[o];
        const int n0 = sh.op_n0[o], no = sh.op_no[o];
        unsigned long long* const tl = p.timeline ? p.timeline + ((size_t)c * LB_CHAIN_MAX_OPS + o) * 8 : nullptr;
        if (tl && tid == 0) { sh.stamp[0] = ch_globaltimer(); sh.stamp[1] = ch_clock(); }
        // ---- grid barrier: every result of entry o-1 is in memory before it is read (a GEMV fed through a mailbox waits on
        //      the words themselves instead).  The block arrives first, then does what it may do before the others have
        //      arrived, then waits. ----
        const bool barrier = o > 0 && !(op.type == LB_CHAIN_OP_GEMV && op.x_src);
        if (barrier) {
            CH_SYNC();
            // arrive with release: this block's results, ordered before by the block barrier, become visible to whoever observes the count
            if (tid == 0) asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(p.sync) : "memory");
        }
        // a mixer entry reads its parameter block and the token position (neither written by this launch) ...
        int dn_pos = 0;
        if (op.type == LB_CHAIN_OP_DELTANET) dn_pos = reinterpret_cast<const lb_dn_layer_params*>(op.ext)->pos[0];
        // ... and a GEMV whose input goes through the per-head norm takes the silu of its gate vector, where it may
        float gz[2][8];
        if (op.type == LB_CHAIN_OP_GEMV && op.x_mode == LB_X_F32_HEADNORM_SILU && op.early_gate) {
            ch_gate_rows(op, tid, op.K / 8, gz[0]);
            ch_gate_rows(op, tid + LB_CHAIN_THREADS, op.K / 8, gz[1]);
        }
        if (barrier) {
            if (tid == 0) {
                // poll with acquire; the status word of an earlier failed wait is looked at only once the wait is already long
                const unsigned target = (unsigned)(++n_barriers) * (unsigned)G;
                bool ok = sh.bad == 0;
                if (ok && ld_acquire_gpu(p.sync) < target) {
                    const uint64_t t0 = globaltimer_ns(), limit = lb_wait_limit_ns(p.status);
                    ok = false;
                    for (unsigned it = 0; it < LB_WAIT_SPINS; ++it) {
                        if (ld_acquire_gpu(p.sync) >= target) { ok = true; break; }
                        if ((it & 255u) == 255u &&
                            (globaltimer_ns() - t0 > limit || *reinterpret_cast<volatile uint32_t*>(p.status) != 0u))
                            break;
                    }
                }
                if (!ok) { atomicCAS(p.status, 0u, LB_DEV_TIMEOUT_COUNTER); sh.bad = 1; }
                sh.snap = *reinterpret_cast<volatile uint32_t*>(&sh.bad);
            }
            CH_SYNC();
        }
        if (tl && tid == 0) sh.stamp[2] = ch_clock();
        if (o == p.trigger_op) pdl_launch_dependents();
        if (sh.snap) break; // uniform: written before the barrier above, by one thread

        if (op.type == LB_CHAIN_OP_DELTANET) {
            // ---- the DeltaNet mixer of a layer: (value head, 32-column slab) units, one per team of 128 threads.
            //      The warps' weight rings stay full meanwhile (their next stages belong to the following GEMV). ----
            const lb_dn_layer_params& dn = *reinterpret_cast<const lb_dn_layer_params*>(op.ext);
            const int team = tid >> 7, tt = tid & (DN_THREADS - 1), NU = dn.HV * (DN_D / DN_COLS);
            dn_unit_smem& sm = reinterpret_cast<dn_unit_smem*>(red)[team];
            auto team_sync = [team] { asm volatile("bar.sync %0, %1;" ::"r"(team + 1), "n"(DN_THREADS) : "memory"); };
            const int pos = dn_pos;
            if (NU <= 2 * G) {
                // At most one unit for each of teams 0 and 1.  Teams 2 and 3 have none: they compute the two 5120-long gate
                // dot products of those units' heads (in_proj_a: team 2, in_proj_b: team 3) while teams 0 and 1 are busy with
                // the convolution and the state, and hand them over through shared memory (named barriers 5 and 6: the
                // consumer waits, the two helper teams only arrive).
                if (team < 2) {
                    const int u = c + G * team;
                    if (u < NU)
                        deltanet_layer_unit<false, true>(dn, u / (DN_D / DN_COLS), u % (DN_D / DN_COLS), tt, sm, team_sync, pos, sh.dn_ab[team], [team] {
                            asm volatile("bar.sync %0, %1;" ::"r"(5 + team), "n"(3 * DN_THREADS) : "memory");
                        });
                } else {
                    for (int k = 0; k < 2; ++k) {
                        const int u = c + G * k;
                        if (u >= NU) break;
                        const int h = u / (DN_D / DN_COLS);
                        float v, unused;
                        dn_gate_dot<1>(dn, (team == 2 ? dn.proj_a : dn.proj_b) + (size_t)h * dn.hidden, nullptr, tt, v, unused);
                        v = dn_unit_sum(v, sm.red, tt, team_sync);
                        if (tt == 0) sh.dn_ab[k][team - 2] = v;
                        asm volatile("bar.arrive %0, %1;" ::"r"(5 + k), "n"(3 * DN_THREADS) : "memory");
                    }
                }
            } else {
                for (int u = c + G * team; u < NU; u += G * (LB_CHAIN_THREADS / DN_THREADS)) {
                    deltanet_layer_unit<false, false>(dn, u / (DN_D / DN_COLS), u % (DN_D / DN_COLS), tt, sm, team_sync, pos, nullptr, [] {});
                    team_sync(); // the unit's shared memory is reused
                }
            }
            if (tid == 0) sh.snap = *reinterpret_cast<volatile uint32_t*>(&sh.bad);
            CH_SYNC();
            if (tl && tid == 0) {
                const unsigned long long now = ch_clock();
                tl[0] = sh.stamp[0]; tl[1] = sh.stamp[1]; tl[2] = sh.stamp[2];
                tl[3] = tl[4] = tl[5] = tl[6] = tl[7] = now;
            }
            if (sh.snap) break;
            continue;
        }

        // ---- the activation vector as exact integers: three signed base-256 digit planes ----
        const unsigned long long* in_mail = op.x_src ? p.mail + (size_t)(op.x_src - 1) * LB_CHAIN_MAIL_WORDS : nullptr;
        const uint32_t in_tag = tag_base + (uint32_t)op.x_src;
        const float unit = op.K <= 8 * LB_CHAIN_THREADS * 2 ? ch_prologue<2>(op, sh, xtab, tid, c == 0, in_mail, in_tag, p.status, tl, gz)
                                                             : ch_prologue<5>(op, sh, xtab, tid, c == 0, in_mail, in_tag, p.status, tl, gz);

        // the residual value this thread will add its column's result to: asked for now, so that the epilogue does not wait for it
        // (nobody else writes the column; this thread's own earlier store is what L2 holds)
        float y_old = 0.f;
        if ((op.y_mode == LB_Y_F32_ACCUM || op.y_mode == LB_Y_TP_ALLREDUCE) && tid < no * 8)
            y_old = __ldcg(reinterpret_cast<const float*>(op.y) + n0 * 8 + tid);
        if (tl && tid == 0) sh.stamp[4] = ch_clock();
        // ---- the stages of GEMV o that this warp took.  Every stage leaves its 16 column sums in its own slot of `red`. ----
        const int nch = sh.op_nch[o];
        for (;;) {
            const uint32_t desc = *reinterpret_cast<volatile uint32_t*>(&wdesc[use_slot]);
            if (desc == CH_NO_STAGE || (int)(desc & 31u) != o) break; // nothing left, or the warp's next stage belongs to a later GEMV
            if (!__all_sync(0xffffffffu, mbar_wait(&wfull[use_slot], use_par))) { // the same answer in every lane
                if (lane == 0) { atomicCAS(p.status, 0u, LB_DEV_TIMEOUT_FULL); sh.bad = 1; }
                break;
            }
            const int pair = (int)((desc >> 5) & 31u), g0 = (int)((desc >> 10) & 4095u), gcount = (int)((desc >> 22) & 7u);
            const unsigned char* stage = ring + (size_t)use_slot * LB_CHAIN_STAGE_BYTES;
            const unsigned char* xg = xtab + (size_t)g0 * CH_XG;
            const bool full_pair = (desc >> 25) & 1u;
            float acc_a = 0.f, acc_b = 0.f;
            // the slot goes back to the copy engine as soon as every lane has its words: refilled with the next stage nobody
            // has asked for (maybe of a later GEMV); its descriptor, written by lane 0, is read after the __syncwarp below.
            // (The lanes' loads from the slot are ahead of the request in the same in-order pipe: the shared-memory atomic
            // that picks the next stage returns after them, and the copy it leads to lands a memory latency later.)
            auto hand_back = [&]() {
                if (++use_slot == (uint32_t)NS) { use_slot = 0; use_par ^= 1u; }
                __syncwarp();
                request();
            };
            if (gcount == CH_GC) {
                if (full_pair) {
                    ch_stage_regs<true> R;
                    R.load(stage, L);
                    hand_back();
                    R.compute(xg, L, acc_a, acc_b);
                } else {
                    ch_stage_regs<false> R;
                    R.load(stage, L);
                    hand_back();
                    R.compute(xg, L, acc_a, acc_b);
                }
            } else {
                if (full_pair) ch_stage_tail<true>(stage, xg, gcount, L, acc_a, acc_b);
                else ch_stage_tail<false>(stage, xg, gcount, L, acc_a, acc_b);
                hand_back();
            }
            acc_a *= L.mul; // digit plane t of the column: its power of 256
            acc_b *= L.mul;
            acc_a += __shfl_xor_sync(0xffffffffu, acc_a, 1);
            acc_b += __shfl_xor_sync(0xffffffffu, acc_b, 1);
            acc_a += __shfl_xor_sync(0xffffffffu, acc_a, 2);
            acc_b += __shfl_xor_sync(0xffffffffu, acc_b, 2);
            if (ft == 0) {
                float* row = red + (size_t)(pair * nch + g0 / CH_GC) * 16;
                row[fg] = acc_a;
                row[8 + fg] = acc_b;
            }
            __syncwarp();
        }
        CH_SYNC();
        if (tl && tid == 0) sh.stamp[5] = ch_clock(); // every stage of the strip consumed

        // ---- column sums over the warps, in warp order; epilogue ----
        const int ncol = no * 8;
        unsigned long long* const out_mail = p.mail + (size_t)o * LB_CHAIN_MAIL_WORDS;
        const uint32_t out_tag = tag_base + (uint32_t)o + 1u;
        if (tid < ncol) {
            const int oct = tid >> 3, g = tid & 7;
            const float* col = red + (size_t)(oct >> 1) * nch * 16 + (oct & 1) * 8 + g;
            float v = 0.f;
#pragma unroll 4
            for (int ch = 0; ch < nch; ++ch) v += col[ch * 16]; // in the order of K
            v *= unit;
            if (tl && tid == 0) sh.stamp[6] = ch_clock() + (v == 1.2345e-30f ? 1 : 0); // the column sum is there
            if (op.y_mode == LB_Y_SWIGLU_F16) {
                sh.vals[tid] = v;
            } else if (op.y_mode == LB_Y_TP_ALLREDUCE) {
                // This rank's partial sum of column n of a row-parallel projection.  (value, generation) goes as ONE 8-byte
                // store into every rank's word array (posted stores over NVLink; the local copy is one of them); then this
                // thread -- which owns column n on every rank -- polls its own rank's array until all ranks' words carry this
                // generation, and adds them in rank order into the residual stream.  Slots alternate with the generation: a
                // rank can only be one exchange ahead of its slowest peer, because it needs that peer's word to finish.
                const lb_tp_params& tp = *reinterpret_cast<const lb_tp_params*>(op.ext);
                const unsigned gen = ar_gen0 + (unsigned)ar_done + 1u;
                const int n = n0 * 8 + tid;
                const size_t slot_at = (size_t)(gen & 1u) * tp.size * tp.n_max + (size_t)n;
                const unsigned long long word = ((unsigned long long)gen << 32) | (unsigned long long)__float_as_uint(v);
#pragma unroll
                for (int r = 0; r < LB_TP_MAX; ++r)
                    if (r < tp.size) st_volatile_u64(tp.words[r] + slot_at + (size_t)tp.rank * tp.n_max, word);
                float sum = 0.f;
                bool ok = sh.bad == 0;
                const uint64_t t0 = globaltimer_ns(), limit = lb_wait_limit_ns(p.status);
#pragma unroll
                for (int r = 0; r < LB_TP_MAX; ++r) {
                    if (r >= tp.size || !ok) continue;
                    const unsigned long long* src = tp.words[tp.rank] + slot_at + (size_t)r * tp.n_max;
                    unsigned long long w = ld_volatile_u64(src);
                    if ((unsigned)(w >> 32) != gen) {
                        ok = false;
                        for (unsigned it = 0; it < LB_WAIT_SPINS; ++it) {
                            w = ld_volatile_u64(src);
                            if ((unsigned)(w >> 32) == gen) { ok = true; break; }
                            if ((it & 63u) == 63u && (globaltimer_ns() - t0 > limit || *reinterpret_cast<volatile uint32_t*>(p.status) != 0u)) break;
                        }
                    }
                    sum += __uint_as_float((unsigned)w); // rank order
                }
                if (ok) {
                    const float nx = y_old + sum;
                    reinterpret_cast<float*>(op.y)[n] = nx;
                    if (op.mail) st_volatile_u64(out_mail + n, ((unsigned long long)out_tag << 32) | __float_as_uint(nx));
                } else { atomicCAS(p.status, 0u, LB_DEV_TIMEOUT_PEER); sh.bad = 1; }
            } else {
                const int n = n0 * 8 + tid;
                if (op.y_mode == LB_Y_F16) reinterpret_cast<__half*>(op.y)[n] = __float2half_rn(v);
                else {
                    const float nx = op.y_mode == LB_Y_F32 ? v : y_old + v;
                    reinterpret_cast<float*>(op.y)[n] = nx;
                    if (op.mail) st_volatile_u64(out_mail + n, ((unsigned long long)out_tag << 32) | __float_as_uint(nx));
                }
            }
        }
        if (op.y_mode == LB_Y_SWIGLU_F16) {
            // the strip is made of (gate octet, up octet) pairs; pair P of the matrix gives y[8P .. 8P+7]
            CH_SYNC();
            if (tid < ncol / 4) { // two neighbouring results per thread: one 4-byte store, one mailbox word
                const int i0 = 2 * tid, pr = i0 >> 3, g = i0 & 7;
                const float a = siluf_dev(sh.vals[pr * 16 + g]) * sh.vals[pr * 16 + 8 + g];
                const float b = siluf_dev(sh.vals[pr * 16 + g + 1]) * sh.vals[pr * 16 + 8 + g + 1];
                const __half2 h = __floats2half2_rn(a, b);
                const int at = (n0 / 2) * 8 + i0;
                *reinterpret_cast<__half2*>(reinterpret_cast<__half*>(op.y) + at) = h;
                if (op.mail) st_volatile_u64(out_mail + (at >> 1), ((unsigned long long)out_tag << 32) | *reinterpret_cast<const uint32_t*>(&h));
            }
        }
        if (op.y_mode == LB_Y_TP_ALLREDUCE) ++ar_done; // one more exchange of this launch (uniform)
        if (tl && tid == 0) {
            sh.stamp[7] = ch_clock();
#pragma unroll
            for (int k = 0; k < 8; ++k) tl[k] = sh.stamp[k];
        }
        if (tid == 0) sh.snap = *reinterpret_cast<volatile uint32_t*>(&sh.bad);
        CH_SYNC(); // red / vals are reused by the next GEMV; sh.snap is the same for everyone
        if (sh.snap) break;
    }
    // ---- leave: the last CTA out zeroes the barrier words for the next launch ----
    CH_SYNC();
    if (tid == 0) {
        __threadfence();
        const unsigned old = atomicAdd(p.sync + 1, 1u);
        if (old == (unsigned)G - 1u) {
            p.sync[0] = 0u;
            p.sync[1] = 0u;
            p.sync[2] = tag_base + LB_CHAIN_MAX_OPS;
            if (ar_tp) const_cast<lb_tp_params*>(ar_tp)->gen[0] = ar_gen0 + (unsigned)ar_done; // every CTA has read the old value
        }
    }
    // no copy may still be in flight into this CTA's shared memory when it exits (only after a failed wait can
    // requested stages be left unconsumed)
    __syncwarp();
    for (int i = 0; i < NS; ++i) {
        if (*reinterpret_cast<volatile uint32_t*>(&wdesc[use_slot]) != CH_NO_STAGE) mbar_wait(&wfull[use_slot], use_par);
        if (++use_slot == (uint32_t)NS) { use_slot = 0; use_par ^= 1u; }
    }
}

// ---------------------------------------------------------------------------
// Reference format (qweight [K/8,N], scales [K/128,N], qzeros [K/128,N/8]) -> strip-packed records
// for G CTAs (layout in params.h).  One thread per 32-bit word of the output; run once per matrix.
// With swiglu set, the input columns are the interleaved 64-wide (gate, up) blocks of the
// LB_Y_SWIGLU_F16 contract and unit P of the output is (gate octet, up octet) of y[8P .. 8P+7].
// ---------------------------------------------------------------------------
extern "C" __global__ void gemv_pack_strips(const __grid_constant__ lb_pack_params p) {
    const int KG = p.K / LB_GEMV_GROUP, NO = p.N / 8;
    const int upo = p.swiglu ? 2 : 1, units = NO / upo;
    const int RW = LB_CHAIN_RECORD / 4; // words per record
    const long long total = (long long)NO * KG * RW;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int word = (int)(i % RW);
        const long long r = i / RW;
        const int O = (int)(r / KG), q = (int)(r % KG); // global octet, K-group
        int lo = 0, hi = p.G; // the CTA whose strip holds octet O: largest c with start(c) <= O
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if ((int)((long long)mid * units / p.G) * upo <= O) lo = mid; else hi = mid;
        }
        const int n0 = (int)((long long)lo * units / p.G) * upo, no = (int)((long long)(lo + 1) * units / p.G) * upo - n0;
        const int oi = O - n0, pair = oi >> 1;
        const int recw = (2 * pair + 1 < no ? 2 : 1) * RW; // words of one K-group of this pair
        const size_t dst = ((size_t)n0 * KG + (size_t)pair * KG * 2) * RW + (size_t)q * recw + (size_t)(oi & 1) * RW + word;
        int col0; // source columns of octet O
        if (p.swiglu) {
            const int P = O >> 1, blk = P >> 3;
            col0 = blk * 128 + (O & 1) * 64 + (P & 7) * 8;
        } else col0 = O * 8;
        uint32_t out;
        if (word < 128) {
            const int lane = word >> 2, j = word & 3, g = lane >> 2, t = lane & 3;
            out = p.qweight[(size_t)(q * LB_GEMV_ROWS + t + 4 * j) * p.N + col0 + g];
        } else {
            const int g = word - 128;
            const uint32_t sc = p.scales[(size_t)q * p.N + col0 + g];
            const uint32_t z = p.qzeros ? (p.qzeros[(size_t)q * (p.N / 8) + (col0 >> 3)] >> (4 * g)) & 0xFu : 8u;
            out = sc | ((uint32_t)__half_as_ushort(__float2half_rn((float)z)) << 16);
        }
        p.out[dst] = out;
    }
}
