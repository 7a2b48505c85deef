// A chain of GPTQ int4 GEMVs in ONE persistent launch on sm_100a.
//
// The decode step of the reference runs its projections as separate launches
// (src/launcher.s:1226-1535, one launch_gemv per projection); at batch 1 each of them moves
// 25-90 MB and a B200 drains that in 4-14 us, so launch gaps, pipeline fill and the split-K tail
// of every launch cost as much as the streaming itself.  Here the GEMVs between two token-mixer
// kernels (out projection, gate/up projection with SwiGLU, down projection, next layer's input
// projection) are one launch of one CTA per SM:
//   * Work of GEMV i = units (column tile of 256, K-group of 128), tile-major; CTA c owns the
//     contiguous unit range [c*U/G, (c+1)*U/G), so every CTA streams the same number of bytes.
//   * One producer lane per CTA feeds a ring of 17 KB stages (16 KB of packed weights, the
//     group's 256 scales, its 32 zero-point words) with tiled TMA loads.  Weights are constants:
//     the producer never waits for a grid barrier, it runs on into the NEXT GEMV's units while
//     the consumers finish the current one.  The ring of all SMs (about 25 MB) is the prefetch
//     buffer that keeps HBM busy across GEMV boundaries.
//   * Consumers (groups of 4 warps, one unit at a time per group) use the same exact integer
//     tensor-core dot product as gemv_int4_w256 (gemv_core.cuh).
//   * A tile split between CTAs is summed in a fixed order: every contributor stores its
//     partial, the last one to arrive (a counter per tile) adds the partials in CTA order and
//     runs the epilogue.  Results do not depend on arrival order.
//   * Between GEMVs the consumers meet at a grid barrier (an arrival counter in global memory,
//     bounded spin).  All CTAs are resident because the grid is one CTA per SM and a CTA takes
//     more than half of an SM's shared memory.
// Activations written inside the launch are read through L2 only (ld.global.cg).
#include "gemv_core.cuh"

#define CH_NG LB_CHAIN_GROUPS
#define CH_CONSUMERS (CH_NG * 128)

__device__ __forceinline__ void ch_bar() { asm volatile("bar.sync 1, %0;" ::"n"(CH_CONSUMERS) : "memory"); }
__device__ __forceinline__ unsigned ld_acquire_gpu(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ long long ch_start(int c, int U, int G) { return (long long)c * U / G; }
// the CTA whose range holds unit u (ranges are non-empty: U >= G is checked by the host)
__device__ __forceinline__ int ch_owner(long long u, int U, int G) { return (int)(((u + 1) * G - 1) / U); }

struct __align__(16) ch_shared {
    float red[CH_NG][LB_GEMV_TILE_N]; // first: written with 16-byte stores
    float scratch[48];
    int xsum[LB_CHAIN_XCAP];
    uint32_t bad;  // a bounded wait ran out (set by any thread at any time)
    uint32_t snap; // copy of bad taken by thread 0 before a consumer barrier: the value all consumers act on together
    uint32_t last; // this CTA delivered the last part of the current tile
};

extern "C" __global__ void __launch_bounds__(LB_CHAIN_THREADS, 1) gemv_chain(const __grid_constant__ lb_chain_params p) {
    extern __shared__ unsigned char smem_raw[];
    __shared__ ch_shared sh;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int c = blockIdx.x, G = gridDim.x;
    const int S = p.stages;

    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    unsigned char* smem = smem_raw + (smem_base - smem_u32(smem_raw));
    uint32_t* xdig = reinterpret_cast<uint32_t*>(smem + (size_t)S * LB_CHAIN_STAGE_STRIDE); // digit table, LB_CHAIN_XCAP groups
    const int dig_words = (digit_row_word(LB_CHAIN_XCAP * LB_GEMV_ROWS) + 3) & ~3;
    uint64_t* full = reinterpret_cast<uint64_t*>(xdig + dig_words);
    uint64_t* empty = full + S;

    if (tid == 0) {
        for (int s = 0; s < S; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 4); // the four warps of the group that consumed the stage
        }
        sh.bad = 0;
        sh.snap = 0;
        sh.last = 0;
        mbar_fence_init();
    }
    __syncthreads();

    uint32_t issued = 0; // producer lane: stages handed to the TMA engine
    if (warp == CH_NG * 4) {
        // ---------------- producer: runs through every GEMV of the chain without stopping ----------------
        if (lane == 0) {
            const uint64_t pol = l2_policy_evict_first();
            bool ok = true;
            for (int o = 0; o < p.n_ops && ok; ++o) {
                const lb_chain_op& op = p.op[o];
                const long long u0 = ch_start(c, op.units, G), u1 = ch_start(c + 1, op.units, G);
                const uint32_t bytes = LB_GEMV_STAGE_BYTES + 512u + (op.has_zeros ? 128u : 0u);
                for (long long u = u0; u < u1; ++u, ++issued) {
                    const int s = issued % S;
                    if (issued >= (uint32_t)S && !mbar_wait(&empty[s], ((issued / S) - 1) & 1)) {
                        atomicExch(p.status, LB_DEV_TIMEOUT_EMPTY);
                        sh.bad = 1;
                        ok = false;
                        break;
                    }
                    if (*reinterpret_cast<volatile uint32_t*>(&sh.bad)) { ok = false; break; }
                    const int tile = (int)(u / op.kg), g = (int)(u - (long long)tile * op.kg);
                    const uint32_t dst = smem_base + (uint32_t)s * LB_CHAIN_STAGE_STRIDE;
                    mbar_arrive_expect_tx(&full[s], bytes); // parts of a box past the matrix are zero-filled and counted
                    tma_load_2d(dst + LB_CHAIN_SCALE_OFF, op.tmap_sc, tile * LB_GEMV_TILE_N, g, &full[s], pol);
                    if (op.has_zeros) tma_load_2d(dst + LB_CHAIN_ZERO_OFF, op.tmap_zr, tile * (LB_GEMV_TILE_N / 8), g, &full[s], pol);
                    tma_load_stage(dst, op.tmap, tile * (LB_GEMV_TILE_N / 32), g * LB_GEMV_ROWS, &full[s], pol);
                }
            }
        }
    } else {
        // ---------------- consumers ----------------
        const int grp = warp >> 2, w4 = warp & 3;
        const int fg = lane >> 2, ft = lane & 3;
        const int cbase = w4 * 64; // this warp's first column inside the tile
        const float lane_mul = ft == 0 ? 1.0f : (ft == 1 ? 65536.0f : 0.0f);
        const bool has_digits = fg < 3;
        pdl_wait(); // activations, barrier words and tile counters belong to the stream order
        uint32_t it0 = 0; // ring position of this CTA's first unit of the current GEMV
        for (int o = 0; o < p.n_ops; ++o) {
            const lb_chain_op& op = p.op[o];
            const int U = op.units, KG = op.kg;
            const long long u0 = ch_start(c, U, G), u1 = ch_start(c + 1, U, G);
            if (o > 0) {
                // ---- grid barrier: every epilogue of GEMV o-1 is in memory before its results are read ----
                ch_bar();
                if (tid == 0) {
                    __threadfence();
                    atomicAdd(p.sync, 1u);
                    const unsigned target = (unsigned)o * (unsigned)G;
                    const uint64_t t0 = globaltimer_ns();
                    bool ok = false;
                    const bool dead = sh.bad || *reinterpret_cast<volatile uint32_t*>(p.status) != 0u;
                    for (unsigned it = 0; it < LB_WAIT_SPINS && !dead; ++it) {
                        if (ld_acquire_gpu(p.sync) >= target) { ok = true; break; }
                        if ((it & 63u) == 63u && globaltimer_ns() - t0 > LB_WAIT_NS) break;
                    }
                    if (!ok) { atomicExch(p.status, LB_DEV_TIMEOUT_COUNTER); sh.bad = 1; }
                    __threadfence();
                    sh.snap = *reinterpret_cast<volatile uint32_t*>(&sh.bad);
                }
                ch_bar();
            }
            if (o == p.trigger_op) pdl_launch_dependents();
            if (sh.snap) break; // uniform: written before the barrier above, by one thread

            // ---- activation table of the K-groups this CTA meets: exact integers, three signed base-256 digits ----
            const int cnt = (u1 - u0) >= KG ? KG : (int)(u1 - u0); // groups in the (cyclic) window
            const int gA = cnt == KG ? 0 : (int)(u0 % KG);
            const int rows = cnt * LB_GEMV_ROWS;
            float rinv = 1.0f;
            if (op.x_mode == LB_X_F32_RMSNORM) {
                const float4* xv = reinterpret_cast<const float4*>(op.x);
                float ss = 0.f;
                for (int i = tid; i < op.K / 4; i += CH_CONSUMERS) {
                    const float4 v = __ldcg(xv + i);
                    ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
                }
                ss = warp_sum(ss);
                if (lane == 0) sh.scratch[warp] = ss;
                ch_bar();
                float tot = 0.f;
#pragma unroll
                for (int w = 0; w < CH_NG * 4; ++w) tot += sh.scratch[w];
                rinv = rsqrtf(tot / (float)op.K + op.eps);
                ch_bar();
            }
            float vmax = 0.f;
            for (int rb = 0; rb < rows; rb += CH_CONSUMERS) {
                float v[8];
                const int r = rb + tid;
                const bool live = r < rows;
                int g = gA + (r >> 4);
                if (g >= KG) g -= KG;
                load_x_row<true>(op, live ? g * LB_GEMV_GROUP + (r & 15) * 8 : 0, live, rinv, v);
#pragma unroll
                for (int j = 0; j < 8; ++j) vmax = fmaxf(vmax, fabsf(v[j]));
                if (live) { // parked as fp16 in the row's own digit slot until the scale is known
                    __half2 pk[4] = {__floats2half2_rn(v[0], v[1]), __floats2half2_rn(v[2], v[3]),
                                     __floats2half2_rn(v[4], v[5]), __floats2half2_rn(v[6], v[7])};
                    uint32_t* dst = xdig + digit_row_word(r);
                    const uint32_t* pw = reinterpret_cast<const uint32_t*>(pk);
                    *reinterpret_cast<uint2*>(dst) = make_uint2(pw[0], pw[1]);
                    *reinterpret_cast<uint2*>(dst + 2) = make_uint2(pw[2], pw[3]);
                }
            }
#pragma unroll
            for (int o2 = 16; o2 > 0; o2 >>= 1) vmax = fmaxf(vmax, __shfl_xor_sync(0xffffffffu, vmax, o2));
            if (lane == 0) sh.scratch[16 + warp] = vmax;
            ch_bar();
            vmax = 0.f;
#pragma unroll
            for (int w = 0; w < CH_NG * 4; ++w) vmax = fmaxf(vmax, sh.scratch[16 + w]);
            int shift = 0; // max|x| * 2^shift in [2^21, 2^22); all-zero or non-finite windows use shift 0
            if (vmax > 0.f && vmax < 3.0e38f) shift = 21 - (int)((__float_as_uint(vmax) >> 23) & 0xffu) + 127;
            const float qscale = __uint_as_float((uint32_t)(127 + shift) << 23);
            const float unit = __uint_as_float((uint32_t)(127 - shift) << 23);
            for (int rb = 0; rb < rows; rb += CH_CONSUMERS) {
                const int r = rb + tid;
                const bool live = r < rows;
                float v[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] = 0.f;
                if (live) { // the same thread parked this row above
                    const uint32_t* src = xdig + digit_row_word(r);
                    const uint2 p0 = *reinterpret_cast<const uint2*>(src), p1 = *reinterpret_cast<const uint2*>(src + 2);
                    const uint32_t pw[4] = {p0.x, p0.y, p1.x, p1.y};
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&pw[j]));
                        v[2 * j] = f.x;
                        v[2 * j + 1] = f.y;
                    }
                }
                int rs = 0;
                uint32_t ev[3] = {0u, 0u, 0u}, od[3] = {0u, 0u, 0u};
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    int t = __float2int_rn(v[j] * qscale);
                    rs += t;
#pragma unroll
                    for (int d = 0; d < 3; ++d) {
                        const int dg = d < 2 ? ((t + 128) & 255) - 128 : t; // signed digit in [-128,127]
                        t = (t - dg) >> 8;
                        const uint32_t byte = (uint32_t)dg & 0xffu;
                        if (j & 1) od[d] |= byte << (8 * (j >> 1));
                        else ev[d] |= byte << (8 * (j >> 1));
                    }
                }
#pragma unroll
                for (int o2 = 8; o2 > 0; o2 >>= 1) rs += __shfl_xor_sync(0xffffffffu, rs, o2); // the group's 16 rows
                if (live) {
                    uint32_t* dst = xdig + digit_row_word(r);
#pragma unroll
                    for (int d = 0; d < 3; ++d) *reinterpret_cast<uint2*>(dst + 2 * d) = make_uint2(ev[d], od[d]);
                    if ((lane & 15) == 0) sh.xsum[r >> 4] = rs;
                    int g = gA + (r >> 4);
                    if (g >= KG) g -= KG;
                    if (op.x_out && g >= u0 && g < u1) { // the CTAs that own units of tile 0 write the vector out once
                        __half2 pl[4] = {__floats2half2_rn(v[0], v[1]), __floats2half2_rn(v[2], v[3]),
                                         __floats2half2_rn(v[4], v[5]), __floats2half2_rn(v[6], v[7])};
                        *reinterpret_cast<uint4*>(op.x_out + g * LB_GEMV_GROUP + (r & 15) * 8) = *reinterpret_cast<uint4*>(pl);
                    }
                }
            }
            ch_bar();

            // ---- this CTA's units, one tile segment at a time ----
            long long ua = u0;
            while (ua < u1 && !sh.snap) {
                const int tile = (int)(ua / KG);
                const long long tile_u0 = (long long)tile * KG;
                const long long ub = u1 < tile_u0 + KG ? u1 : tile_u0 + KG;
                const int n0 = tile * LB_GEMV_TILE_N;
                const int ncols = min(LB_GEMV_TILE_N, op.N - n0);
                const bool live0 = cbase < ncols, live1 = cbase + 32 < ncols; // N % 32 == 0
                float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
                // group grp takes the units whose ring position is grp modulo the number of groups
                const uint32_t pos_a = it0 + (uint32_t)(ua - u0);
                const int off = (grp + CH_NG - (int)(pos_a % CH_NG)) % CH_NG;
                for (long long u = ua + off; u < ub; u += CH_NG) {
                    const uint32_t idx = it0 + (uint32_t)(u - u0);
                    const int s = idx % S;
                    int slot = (int)(u - tile_u0) - gA; // position of the K-group in the activation table
                    if (slot < 0) slot += KG;
                    if (!mbar_wait(&full[s], (idx / S) & 1)) {
                        if (lane == 0) { atomicExch(p.status, LB_DEV_TIMEOUT_FULL); sh.bad = 1; }
                        break;
                    }
                    const unsigned char* stage = smem + (size_t)s * LB_CHAIN_STAGE_STRIDE;
                    uint2 sraw[2];
                    uint32_t zw[2];
                    sraw[0] = *reinterpret_cast<const uint2*>(stage + LB_CHAIN_SCALE_OFF + (cbase + fg * 4) * 2);
                    sraw[1] = *reinterpret_cast<const uint2*>(stage + LB_CHAIN_SCALE_OFF + (cbase + 32 + fg * 4) * 2);
                    zw[0] = zw[1] = 0x88888888u;
                    if (op.has_zeros) {
                        zw[0] = *reinterpret_cast<const uint32_t*>(stage + LB_CHAIN_ZERO_OFF + ((cbase + fg * 4) >> 3) * 4);
                        zw[1] = *reinterpret_cast<const uint32_t*>(stage + LB_CHAIN_ZERO_OFF + ((cbase + 32 + fg * 4) >> 3) * 4);
                    }
                    int d[2][2][4]; // [box][column pair][fragment]
#pragma unroll
                    for (int i = 0; i < 16; ++i) (&d[0][0][0])[i] = 0;
                    if (live0) {
                        const unsigned char* box = stage + (w4 * 2) * GEMV_BOX_BYTES;
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const int r = 8 * (e >> 1) + 2 * ft + (e & 1);
                            uint2 xb = make_uint2(0u, 0u);
                            if (has_digits) xb = *reinterpret_cast<const uint2*>(xdig + digit_row_word(slot * LB_GEMV_ROWS + r) + 2 * fg);
                            const uint32_t boff = r * 128 + ((fg ^ (r & 7)) << 4);
                            const uint4 w0 = *reinterpret_cast<const uint4*>(box + boff);
                            imma_words(d[0][0], w0.x, w0.y, xb);
                            imma_words(d[0][1], w0.z, w0.w, xb);
                            if (live1) {
                                const uint4 w1 = *reinterpret_cast<const uint4*>(box + GEMV_BOX_BYTES + boff);
                                imma_words(d[1][0], w1.x, w1.y, xb);
                                imma_words(d[1][1], w1.z, w1.w, xb);
                            }
                        }
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&empty[s]); // this warp is done with the stage
                    const float xs_f = ft == 0 ? (float)sh.xsum[slot] : 0.f;
#pragma unroll
                    for (int b = 0; b < 2; ++b) {
                        const float2 s01 = __half22float2(*reinterpret_cast<const __half2*>(&sraw[b].x));
                        const float2 s23 = __half22float2(*reinterpret_cast<const __half2*>(&sraw[b].y));
                        const uint32_t z = zw[b] >> ((fg & 1) * 16);
                        const float sc[4] = {s01.x, s01.y, s23.x, s23.y};
#pragma unroll
                        for (int cc = 0; cc < 4; ++cc) {
                            const int* f = d[b][cc >> 1];
                            const int comb = f[(cc & 1) * 2] + (f[(cc & 1) * 2 + 1] << 8);
                            const float zf = __uint_as_float(0x4B000000u | ((z >> (4 * cc)) & 0xFu)) - 8388608.0f;
                            acc[b * 4 + cc] = fmaf(sc[cc], fmaf(-zf, xs_f, (float)comb * lane_mul), acc[b * 4 + cc]);
                        }
                    }
                }
                // ---- segment done: the groups' sums, in group order ----
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    float a = acc[i];
                    a += __shfl_xor_sync(0xffffffffu, a, 1);
                    a += __shfl_xor_sync(0xffffffffu, a, 2);
                    acc[i] = a * unit;
                }
                if (ft == 0) {
                    *reinterpret_cast<float4*>(&sh.red[grp][cbase + fg * 4]) = make_float4(acc[0], acc[1], acc[2], acc[3]);
                    *reinterpret_cast<float4*>(&sh.red[grp][cbase + 32 + fg * 4]) = make_float4(acc[4], acc[5], acc[6], acc[7]);
                }
                ch_bar();
                const bool owner = tid < LB_GEMV_TILE_N;
                float v = 0.f;
                if (owner) {
#pragma unroll
                    for (int gq = 0; gq < CH_NG; ++gq) v += sh.red[gq][tid];
                }
                bool run_epilogue = true;
                if (ub - ua < KG) {
                    // the tile is shared: deliver this part; the last contributor adds all parts in CTA order
                    const int first = ch_owner(tile_u0, U, G), lastc = ch_owner(tile_u0 + KG - 1, U, G);
                    const int myslot = tile == (int)(u0 / KG) ? 0 : 1;
                    if (owner) __stcg(p.partial + ((size_t)c * 2 + myslot) * LB_GEMV_TILE_N + tid, v);
                    __threadfence();
                    ch_bar();
                    if (tid == 0) {
                        const unsigned old = atomicAdd(p.tile_count + tile, 1u);
                        const bool last = old == (unsigned)(lastc - first);
                        if (last) p.tile_count[tile] = 0u; // everybody has arrived: ready for the next GEMV
                        sh.last = last ? 1u : 0u;
                    }
                    ch_bar();
                    run_epilogue = sh.last != 0u;
                    if (run_epilogue && owner) {
                        __threadfence();
                        v = 0.f;
                        for (int cc = first; cc <= lastc; ++cc) {
                            const int sl = tile == (int)(ch_start(cc, U, G) / KG) ? 0 : 1;
                            v += __ldcg(p.partial + ((size_t)cc * 2 + sl) * LB_GEMV_TILE_N + tid);
                        }
                    }
                }
                if (run_epilogue) {
                    if (op.y_mode == LB_Y_SWIGLU_F16) {
                        // columns come in interleaved 64-wide (gate, up) blocks: [0,64) gate, [64,128) up, ...
                        ch_bar();
                        if (owner) sh.red[0][tid] = v;
                        ch_bar();
                        if (tid < ncols / 2) {
                            const int blk = tid >> 6, i = tid & 63;
                            const float gate = sh.red[0][blk * 128 + i], up = sh.red[0][blk * 128 + 64 + i];
                            reinterpret_cast<__half*>(op.y)[n0 / 2 + tid] = __float2half_rn(siluf_dev(gate) * up);
                        }
                    } else if (owner && tid < ncols) {
                        const int n = n0 + tid;
                        if (op.y_mode == LB_Y_F16) reinterpret_cast<__half*>(op.y)[n] = __float2half_rn(v);
                        else if (op.y_mode == LB_Y_F32) reinterpret_cast<float*>(op.y)[n] = v;
                        else reinterpret_cast<float*>(op.y)[n] = __ldcg(reinterpret_cast<float*>(op.y) + n) + v;
                    }
                }
                if (tid == 0) sh.snap = *reinterpret_cast<volatile uint32_t*>(&sh.bad);
                ch_bar(); // sh.red and sh.last are reused by the next segment; sh.snap is the same for everyone
                ua = ub;
            }
            it0 += (uint32_t)(u1 - u0);
        }
        // ---- leave: the last CTA out zeroes the barrier words for the next launch ----
        ch_bar();
        if (tid == 0) {
            __threadfence();
            const unsigned old = atomicAdd(p.sync + 1, 1u);
            if (old == (unsigned)G - 1u) {
                p.sync[0] = 0u;
                p.sync[1] = 0u;
            }
        }
    }
    __syncthreads();
    // after a failed wait: no copy may still be in flight into this CTA's shared memory when it exits
    if (sh.bad && warp == CH_NG * 4 && lane == 0) {
        for (uint32_t k = issued > (uint32_t)S ? issued - S : 0u; k < issued; ++k) mbar_wait(&full[k % S], (k / S) & 1);
    }
}
