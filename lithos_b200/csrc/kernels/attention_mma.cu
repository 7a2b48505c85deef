// GQA decode attention on the tensor cores (sm_100a): same contract, parameter block and results as
// attn_decode_split (attention.cu; inference/attend.ls:85-191, attend_full.ls:186-248), rebuilt around
// two facts measured on that kernel: a K/V row cost about 200 instructions per warp (per-lane dot
// products, 30 shuffles, scalar soft-max for six heads), and every warp had only two rows in flight.
//   * A CTA is (KV head, slice of positions); a warp takes blocks of 16 rows.  The 16 K rows and 16 V
//     rows of a block (512 B each) come by 1-D bulk copies into the warp's own padded tile; the first
//     block of every warp is requested at kernel start, before griddepcontrol.wait (cache rows below
//     the current position are never written by this step).
//   * S = Q K^T as mma.sync.m16n8k16 bf16: A = the query heads of the KV head (rows 0..G-1 of the
//     fragment, the rest zero), B = the K rows.  Q is the normalised, rotated, pre-scaled fp32 query
//     split into two bf16 terms (hi + lo), so the scores carry 16 bits of Q; K is bf16 in the cache.
//   * O^T = V^T P^T: A = V through ldmatrix.trans, B = the probabilities, which come out of the first
//     product in exactly the B-fragment layout (head g, rows 2t and 2t+1); P also as hi + lo.
//   * Online soft-max per head over the warp's blocks, warps merged through shared memory in warp
//     order, slices merged by the last CTA to arrive in slice order: run-to-run identical.
// mma.sync rather than tcgen05: M is the 1..6 query heads of a KV head.
#include "attention_core.cuh"

#define AM_ROWS 16
#define AM_STRIDE 528 // bytes per staged row: 512 + 16, so that 8 rows hit 8 different bank groups
#define AM_TILE (2 * AM_ROWS * AM_STRIDE)

__device__ __forceinline__ void mma_bf16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x2(uint32_t addr, uint32_t& r0, uint32_t& r1) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];" : "=r"(r0), "=r"(r1) : "r"(addr));
}
// (x, y) as a bf16 pair (x in the low half) and the bf16 pair of what the rounding left over
__device__ __forceinline__ void split_bf16x2(float x, float y, uint32_t& hi, uint32_t& lo) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(x, y);
    const float2 hf = __bfloat1622float2(h);
    const __nv_bfloat162 l = __floats2bfloat162_rn(x - hf.x, y - hf.y);
    hi = *reinterpret_cast<const uint32_t*>(&h);
    lo = *reinterpret_cast<const uint32_t*>(&l);
}

template <int G>
__device__ __forceinline__ void attn_mma_body(const lb_attn_params& p0, unsigned char* sm) {
    lb_attn_params p = p0;
    const int kv = blockIdx.x, split = blockIdx.y;
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const int fg = lane >> 2, ft = lane & 3;
    // shared memory
    unsigned char* tiles = sm;                                            // [8 warps][K 16 rows | V 16 rows][528 B]
    float* q_s = reinterpret_cast<float*>(tiles + AT_WARPS * AM_TILE);    // [G][256] fp32 query heads
    unsigned char* qh = reinterpret_cast<unsigned char*>(q_s + G * AT_D); // [8][528 B] bf16 hi
    unsigned char* ql = qh + 8 * AM_STRIDE;                               // [8][528 B] bf16 lo
    float* kn_s = reinterpret_cast<float*>(ql + 8 * AM_STRIDE);           // [256] new key (bf16-rounded)
    float* vn_s = kn_s + AT_D;                                            // [256] new value
    float* cs_s = vn_s + AT_D;                                            // [128]
    float* sn_s = cs_s + 128;                                             // [128]
    float* wm = sn_s + 128;                                               // [8][8] per-warp max
    float* wl = wm + AT_WARPS * AT_GMAX;                                  // [8][8] per-warp sum
    uint64_t* bars = reinterpret_cast<uint64_t*>(wl + AT_WARPS * AT_GMAX); // [8]
    __shared__ uint32_t s_ticket;

    unsigned char* my_tile = tiles + warp * AM_TILE;
    if (lane == 0) mbar_init(&bars[warp], 1);
    mbar_fence_init();
    __syncwarp();

    // The position comes from device memory written by the previous STEP (not the previous kernel), and cache rows
    // below it are not written by this step: the first block of every warp can be requested at once.
    if (p.pos_ptr) p.pos = p.pos_ptr[0];
    if (p.max_ctx > 0 && (p.pos < 0 || p.pos >= p.max_ctx)) { // the position lies outside the caches: report it, touch nothing
        if (threadIdx.x == 0 && blockIdx.x == 0 && blockIdx.y == 0 && p.status) atomicExch(p.status, LB_DEV_POS_RANGE);
        return;
    }
    const int chunk = (((p.pos + p.splits - 1) / p.splits) + AM_ROWS - 1) & ~(AM_ROWS - 1); // rows per slice, whole blocks
    const int t0 = split * chunk, t1 = min(p.pos, t0 + chunk);
    const int n_blocks = t1 > t0 ? (t1 - t0 + AM_ROWS - 1) / AM_ROWS : 0;
    const size_t row_bytes = (size_t)p.HKV * AT_D * 2;
    const uint64_t pol = l2_policy_evict_first();
    auto request = [&](int b) { // rows past the slice end repeat its last row (finite values; their scores are masked)
        if (lane == 0) mbar_arrive_expect_tx(&bars[warp], 2 * AM_ROWS * 512);
        __syncwarp();
        const int r = min(t0 + b * AM_ROWS + (lane & 15), t1 - 1);
        const unsigned char* base = reinterpret_cast<const unsigned char*>(lane < 16 ? p.k_cache : p.v_cache);
        bulk_g2s(my_tile + (lane < 16 ? 0 : AM_ROWS * AM_STRIDE) + (lane & 15) * AM_STRIDE, base + (size_t)r * row_bytes + (size_t)kv * AT_D * 2,
                 512, &bars[warp], pol);
    };
    if (warp < n_blocks) request(warp);

    pdl_wait();
    const bool last = split == p.splits - 1; // this CTA also appends and attends the token being decoded
    const float LOG2E = 1.4426950408889634f;
    const float qscale = rsqrtf((float)AT_D) * LOG2E; // scores kept in log2 units
    // cos/sin of this position once per CTA: the angle is formed and reduced modulo 2*pi in double, the trigonometry
    // itself is fp32 on |r| <= pi; freq comes from the host in double
    if (t < p.rot_dims / 2) {
        const double a = (double)p.pos * p.rope_freq[t];
        const double k = rint(a * 0.15915494309189535);
        const float r = (float)fma(-k, 6.283185307179586, a);
        sincosf(r, &sn_s[t], &cs_s[t]);
    }
    __syncthreads();
    for (int row = warp; row < G + (last ? 1 : 0); row += AT_WARPS) {
        if (row < G)
            warp_norm_rope(p.q, (size_t)(kv * G + row) * p.q_stride, p.in_dtype, p.q_norm_w, q_s + row * AT_D, cs_s, sn_s, p.rot_dims,
                           p.eps, qscale);
        else
            warp_norm_rope(p.k_new, (size_t)kv * AT_D, p.in_dtype, p.k_norm_w, kn_s, cs_s, sn_s, p.rot_dims, p.eps, 1.0f);
    }
    __syncthreads();
    // the query heads as two bf16 terms, rows G..7 zero: thread t owns dim t
#pragma unroll
    for (int g = 0; g < 8; ++g) {
        const float q = g < G ? q_s[g * AT_D + t] : 0.f;
        const __nv_bfloat16 h = __float2bfloat16_rn(q);
        reinterpret_cast<__nv_bfloat16*>(qh + g * AM_STRIDE)[t] = h;
        reinterpret_cast<__nv_bfloat16*>(ql + g * AM_STRIDE)[t] = __float2bfloat16_rn(q - __bfloat162float(h));
    }
    if (last) {
        const __nv_bfloat16 kb = __float2bfloat16_rn(kn_s[t]);
        const __nv_bfloat16 vb = __float2bfloat16_rn(ld_in(p.v_new, (size_t)kv * AT_D + t, p.in_dtype));
        const size_t row = ((size_t)p.pos * p.HKV + kv) * AT_D + t;
        reinterpret_cast<__nv_bfloat16*>(p.k_cache)[row] = kb; // KV append
        reinterpret_cast<__nv_bfloat16*>(p.v_cache)[row] = vb;
        kn_s[t] = __bfloat162float(kb);
        vn_s[t] = __bfloat162float(vb);
    }
    __syncthreads();
    pdl_launch_dependents();

    // ---- this warp's blocks: running (max, sum) of head fg in the four lanes of row group fg, and
    //      O^T[dim][head] in fragment layout: acc[mb] = dims 16mb+fg (c0,c1) and 16mb+8+fg (c2,c3), heads 2ft, 2ft+1 ----
    float m_run = -INFINITY, l_run = 0.f;
    float acc[16][4];
#pragma unroll
    for (int mb = 0; mb < 16; ++mb) acc[mb][0] = acc[mb][1] = acc[mb][2] = acc[mb][3] = 0.f;
    const uint32_t k_addr = smem_u32(my_tile), v_addr = k_addr + AM_ROWS * AM_STRIDE;
    // ldmatrix row addresses.  K (x4): matrices (rows 0-7, dims c..c+7), (rows 0-7, +8), (rows 8-15, c), (rows 8-15, +8).
    const uint32_t k_lane = k_addr + ((lane & 7) + ((lane >> 4) << 3)) * AM_STRIDE + ((lane >> 3) & 1) * 16;
    // V (x4, transposed): matrices (rows 0-7, dims m..m+7), (rows 0-7, +8), (rows 8-15, m), (rows 8-15, +8)
    const uint32_t v_lane = v_addr + ((lane & 7) + ((lane >> 4) << 3)) * AM_STRIDE + ((lane >> 3) & 1) * 16;
    // Q (x2): (heads 0-7, dims c..c+7), (heads 0-7, +8); lanes 16-31 repeat valid addresses
    const uint32_t qh_lane = smem_u32(qh) + (lane & 7) * AM_STRIDE + ((lane >> 3) & 1) * 16;
    const uint32_t ql_lane = smem_u32(ql) + (lane & 7) * AM_STRIDE + ((lane >> 3) & 1) * 16;

    auto block = [&](int nvalid) {
        // S[head][row] = sum over 256 dims, 16 at a time; n-block 0 = rows 0-7, n-block 1 = rows 8-15
        float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int c = 0; c < 16; ++c) {
            uint32_t ah0, ah2, al0, al2, b00, b01, b10, b11;
            ldsm_x2(qh_lane + c * 32, ah0, ah2);
            ldsm_x2(ql_lane + c * 32, al0, al2);
            ldsm_x4(k_lane + c * 32, b00, b01, b10, b11);
            mma_bf16(s0, ah0, 0u, ah2, 0u, b00, b01);
            mma_bf16(s0, al0, 0u, al2, 0u, b00, b01);
            mma_bf16(s1, ah0, 0u, ah2, 0u, b10, b11);
            mma_bf16(s1, al0, 0u, al2, 0u, b10, b11);
        }
        // lane (fg, ft): s0[0], s0[1] = head fg, rows 2ft, 2ft+1; s1[0], s1[1] = rows 8+2ft, 9+2ft
        float sv[4] = {s0[0], s0[1], s1[0], s1[1]};
        const int r0 = 2 * ft;
        if (r0 >= nvalid) sv[0] = -INFINITY;
        if (r0 + 1 >= nvalid) sv[1] = -INFINITY;
        if (r0 + 8 >= nvalid) sv[2] = -INFINITY;
        if (r0 + 9 >= nvalid) sv[3] = -INFINITY;
        float mb_ = fmaxf(fmaxf(sv[0], sv[1]), fmaxf(sv[2], sv[3]));
        mb_ = fmaxf(mb_, __shfl_xor_sync(0xffffffffu, mb_, 1));
        mb_ = fmaxf(mb_, __shfl_xor_sync(0xffffffffu, mb_, 2));
        const float m_new = fmaxf(m_run, mb_); // row 0 of a block is always valid: finite
        const float corr = exp2f(m_run - m_new); // exp2f(-inf) = 0 on the first block
        float pr[4], ps = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            pr[i] = exp2f(sv[i] - m_new);
            ps += pr[i];
        }
        ps += __shfl_xor_sync(0xffffffffu, ps, 1);
        ps += __shfl_xor_sync(0xffffffffu, ps, 2);
        l_run = fmaf(l_run, corr, ps);
        m_run = m_new;
        // P^T as the B operand: b0 = (P[row 2ft][head fg], P[row 2ft+1][head fg]), b1 = rows 8+2ft, 9+2ft
        uint32_t ph0, pl0, ph1, pl1;
        split_bf16x2(pr[0], pr[1], ph0, pl0);
        split_bf16x2(pr[2], pr[3], ph1, pl1);
        // the accumulators of this lane belong to heads 2ft and 2ft+1: their correction factors live in row groups 2ft, 2ft+1
        const float c0 = __shfl_sync(0xffffffffu, corr, (2 * ft) * 4), c1 = __shfl_sync(0xffffffffu, corr, (2 * ft + 1) * 4);
#pragma unroll
        for (int mb = 0; mb < 16; ++mb) {
            uint32_t a0, a1, a2, a3;
            ldsm_x4_trans(v_lane + mb * 32, a0, a1, a2, a3);
            acc[mb][0] *= c0; acc[mb][1] *= c1; acc[mb][2] *= c0; acc[mb][3] *= c1;
            mma_bf16(acc[mb], a0, a1, a2, a3, ph0, ph1);
            mma_bf16(acc[mb], a0, a1, a2, a3, pl0, pl1);
        }
    };

    uint32_t phase = 0;
    for (int b = warp; b < n_blocks; b += AT_WARPS) {
        if (!__all_sync(0xffffffffu, mbar_wait(&bars[warp], phase))) {
            if (lane == 0 && p.status) atomicExch(p.status, LB_DEV_TIMEOUT_FULL);
            break;
        }
        phase ^= 1u;
        block(min(AM_ROWS, t1 - (t0 + b * AM_ROWS)));
        __syncwarp(); // all fragment loads of this block are done: the tile can be refilled
        if (b + AT_WARPS < n_blocks) request(b + AT_WARPS);
    }
    if (last && warp == 0) { // the token being decoded: a block whose 16 rows all repeat it, one of them valid
        __syncwarp();
        uint32_t kw[4], vw[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const __nv_bfloat162 kk = __floats2bfloat162_rn(kn_s[lane * 8 + 2 * j], kn_s[lane * 8 + 2 * j + 1]);
            const __nv_bfloat162 vv = __floats2bfloat162_rn(vn_s[lane * 8 + 2 * j], vn_s[lane * 8 + 2 * j + 1]);
            kw[j] = *reinterpret_cast<const uint32_t*>(&kk);
            vw[j] = *reinterpret_cast<const uint32_t*>(&vv);
        }
#pragma unroll
        for (int r = 0; r < AM_ROWS; ++r) {
            *reinterpret_cast<uint4*>(my_tile + r * AM_STRIDE + lane * 16) = make_uint4(kw[0], kw[1], kw[2], kw[3]);
            *reinterpret_cast<uint4*>(my_tile + (AM_ROWS + r) * AM_STRIDE + lane * 16) = make_uint4(vw[0], vw[1], vw[2], vw[3]);
        }
        __syncwarp();
        block(1);
    }

    // ---- merge the 8 warps (fixed order): per-warp results into the warp's own tile, then thread t owns dim t ----
    __syncwarp();
    float* my_acc = reinterpret_cast<float*>(my_tile); // [G][256]
    if (ft == 0 && fg < G) {
        wm[warp * AT_GMAX + fg] = m_run;
        wl[warp * AT_GMAX + fg] = l_run;
    }
#pragma unroll
    for (int mb = 0; mb < 16; ++mb) {
        if (2 * ft < G) {
            my_acc[(2 * ft) * AT_D + 16 * mb + fg] = acc[mb][0];
            my_acc[(2 * ft) * AT_D + 16 * mb + 8 + fg] = acc[mb][2];
        }
        if (2 * ft + 1 < G) {
            my_acc[(2 * ft + 1) * AT_D + 16 * mb + fg] = acc[mb][1];
            my_acc[(2 * ft + 1) * AT_D + 16 * mb + 8 + fg] = acc[mb][3];
        }
    }
    __syncthreads();
    float Mg[G], Lg[G], Ag[G];
#pragma unroll
    for (int g = 0; g < G; ++g) {
        float M = -INFINITY;
        for (int w = 0; w < AT_WARPS; ++w) M = fmaxf(M, wm[w * AT_GMAX + g]);
        float L = 0.f, A = 0.f;
        for (int w = 0; w < AT_WARPS; ++w) {
            const float mw = wm[w * AT_GMAX + g];
            const float sc = mw == -INFINITY ? 0.f : exp2f(mw - M);
            L = fmaf(wl[w * AT_GMAX + g], sc, L);
            A = fmaf(reinterpret_cast<const float*>(tiles + w * AM_TILE)[g * AT_D + t], sc, A);
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
        if (p.coop) {
            // Every CTA of the launch is resident (the host sets coop only when the grid fits the SMs, one CTA each):
            // all CTAs of this KV head wait for each other and each finishes its own share of the (head, dim)
            // outputs, instead of one CTA doing all of them.
            __syncthreads(); // the whole record is written
            if (t == 0) {
                asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(p.counters + kv) : "memory");
                const uint64_t w0 = globaltimer_ns();
                bool ok = false;
                for (unsigned it = 0; it < LB_WAIT_SPINS; ++it) {
                    unsigned v;
                    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p.counters + kv) : "memory");
                    if (v >= (unsigned)p.splits) { ok = true; break; }
                    if ((it & 255u) == 255u && globaltimer_ns() - w0 > LB_WAIT_NS) break;
                }
                if (!ok && p.status) atomicExch(p.status, LB_DEV_TIMEOUT_COUNTER);
            }
            __syncthreads();
            const float* kvrec = p.scratch + (size_t)kv * p.splits * G * AT_REC;
            const int per = (G * AT_D + p.splits - 1) / p.splits; // outputs of this CTA: [split * per, (split + 1) * per)
            float* pm = reinterpret_cast<float*>(tiles);         // [4][64] partial maxima, sums, accumulators of the four slice groups
            float* pl = pm + 4 * 64;
            float* pa = pl + 4 * 64;
            const int sub = t >> 6, ol = t & 63; // slice group (slices sub, sub + 4, ...), output inside a block of 64
            for (int ob = 0; ob < per; ob += 64) {
                const int o = split * per + ob + ol;
                const bool live = ob + ol < per && o < G * AT_D;
                const int g = live ? o / AT_D : 0, dim = live ? o % AT_D : 0;
                float mv[16], lv[16], av[16];
#pragma unroll
                for (int j = 0; j < 16; ++j) { // up to 64 slices: 16 per group, all loads in flight at once
                    const int s2 = sub + 4 * j;
                    const bool on = live && s2 < p.splits;
                    const float* r = kvrec + ((size_t)(on ? s2 : 0) * G + g) * AT_REC;
                    mv[j] = on ? __ldcg(r + 256) : -INFINITY;
                    lv[j] = on ? __ldcg(r + 257) : 0.f;
                    av[j] = on ? __ldcg(r + dim) : 0.f;
                }
                float M = -INFINITY;
#pragma unroll
                for (int j = 0; j < 16; ++j) M = fmaxf(M, mv[j]);
                float L = 0.f, A = 0.f;
#pragma unroll
                for (int j = 0; j < 16; ++j) { // slice order inside the group
                    const float w = mv[j] == -INFINITY ? 0.f : exp2f(mv[j] - M);
                    L = fmaf(lv[j], w, L);
                    A = fmaf(av[j], w, A);
                }
                __syncthreads(); // the previous block of outputs has been combined
                pm[sub * 64 + ol] = M; pl[sub * 64 + ol] = L; pa[sub * 64 + ol] = A;
                __syncthreads();
                if (sub == 0 && live) { // the four groups, in group order
                    float Mx = fmaxf(fmaxf(pm[ol], pm[64 + ol]), fmaxf(pm[128 + ol], pm[192 + ol]));
                    float Lx = 0.f, Ax = 0.f;
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const float w = pm[q * 64 + ol] == -INFINITY ? 0.f : exp2f(pm[q * 64 + ol] - Mx);
                        Lx = fmaf(pl[q * 64 + ol], w, Lx);
                        Ax = fmaf(pa[q * 64 + ol], w, Ax);
                    }
                    const int hq = kv * G + g;
                    float out = Ax / Lx;
                    if (p.gate) out *= sigmoidf_dev(ld_in(p.gate, (size_t)hq * p.gate_stride + dim, p.in_dtype));
                    p.out[(size_t)hq * AT_D + dim] = out;
                }
            }
            __syncthreads();
            if (t == 0) { // the last CTA to finish reading puts both counters back to zero
                const unsigned old = atomicAdd(p.counters + 8 + kv, 1u);
                if (old == (unsigned)p.splits - 1u) {
                    p.counters[kv] = 0u;
                    p.counters[8 + kv] = 0u;
                }
            }
            return;
        }
        __threadfence();
        __syncthreads();
        if (t == 0) s_ticket = atomicAdd(p.counters + kv, 1u);
        __syncthreads();
        if (s_ticket != (uint32_t)(p.splits - 1)) return;
        __threadfence();
        // all (max, sum) pairs of this KV head in one parallel pass, then the slice weights once
        float* ms_s = reinterpret_cast<float*>(tiles);  // [splits][G] slice maxima, then slice weights (the tiles are free now)
        float* ls_s = ms_s + p.splits * G;              // [splits][G] slice sums
        float* Mx_s = ls_s + p.splits * G;              // [G]
        const float* kvrec = p.scratch + (size_t)kv * p.splits * G * AT_REC;
        __syncthreads();
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
        for (int s2 = 0; s2 < p.splits; s2 += 16) { // 16*G independent loads in flight, then added in slice order
            float a16[G][16];
#pragma unroll
            for (int g = 0; g < G; ++g)
#pragma unroll
                for (int j = 0; j < 16; ++j)
                    a16[g][j] = s2 + j < p.splits ? __ldcg(kvrec + ((size_t)(s2 + j) * G + g) * AT_REC + t) : 0.f;
#pragma unroll
            for (int j = 0; j < 16; ++j)
                if (s2 + j < p.splits) {
#pragma unroll
                    for (int g = 0; g < G; ++g) {
                        const float w = ms_s[(s2 + j) * G + g];
                        Lg[g] = fmaf(ls_s[(s2 + j) * G + g], w, Lg[g]);
                        Ag[g] = fmaf(a16[g][j], w, Ag[g]);
                    }
                }
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

extern "C" __global__ void __launch_bounds__(AT_THREADS, 1) attn_decode_mma(const __grid_constant__ lb_attn_params p) {
    extern __shared__ __align__(128) unsigned char am_sm[];
    const int G = p.HQ / p.HKV;
    switch (G) {
        case 1: attn_mma_body<1>(p, am_sm); break;
        case 2: attn_mma_body<2>(p, am_sm); break;
        case 3: attn_mma_body<3>(p, am_sm); break;
        case 4: attn_mma_body<4>(p, am_sm); break;
        case 6: attn_mma_body<6>(p, am_sm); break;
        default: break; // host rejects other ratios
    }
}
