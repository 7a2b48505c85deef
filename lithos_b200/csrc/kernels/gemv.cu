// GPTQ int4 weight-only GEMV for batch-1 decode on sm_100a.
//
// Replaces the reference's minds/gptq_gemv_safe.ptx (and its v2..v9 siblings,
// inference/gemv.ls) for the primary contract: qweight int32 [K/8,N] (nibble j
// of word (kp,n) is k = 8kp+j), scales fp16 [K/128,N], qzeros int32
// [K/128,N/8] (NULL = zero-point 8, the reference's constant), x fp16, fp32
// accumulation over groups, y fp16/fp32.
//
// Shape of the kernel.  At B200 bandwidth (6.5 TB/s measured) a weight must cost well
// under one instruction or the SMs, not HBM, bound the GEMV: scalar dequant (4 ops/weight
// in the reference), fp16x2 FMA (2.4 ops/weight measured here) and even fp16 mma.sync
// (8 cycles per 256 weights per SM sub-partition) all measured slower than the memory
// stream.  Per-thread loads are too slow as well (about 2.7 TB/s measured for read-only
// ld.global on this part).  So:
//   * Weights are streamed by the TMA engine: CTA (tile, split) owns 256 output columns
//     and a contiguous range of K-groups; one elected producer lane feeds a ring of
//     16 KB stages (one group x 256 columns) with ONE tiled cp.async.bulk.tensor.3d each
//     (eight 32-column boxes, 128-byte swizzle, completion on an mbarrier, L2 evict-first).
//   * The dot products are exact integer arithmetic on the tensor cores:
//     mma.sync.m16n8k32.u8.s8.  A fragment = packed words as they are: w & 0x0f0f0f0f
//     and (w >> 4) & 0x0f0f0f0f (3 instructions per 8 weights); B fragment = the fp16
//     activations scaled by a power of two to integers |X| < 2^22 and split into three
//     signed base-256 digits, one B column per digit plane.  sum q*X is exact in int32;
//     the zero-point term z * sum X, the digit weights, the fp16 group scale and 2^-shift
//     are applied per group in fp32.  X is exact for every activation within 2^-11 of the
//     slice maximum (and off by at most max|x| 2^-23 below), so the result is closer to
//     the real-number dot product than an fp32 FMA loop.
//     (mma.sync rather than tcgen05: M is 1 here; tcgen05's 64/128-row tiles belong to the
//     batched path.  The int4 mma shape is emulated on this part: 152 cycles measured.)
//   * A CTA needs about 55 KB of shared memory, so the CTAs of TWO consecutive kernels
//     fit on an SM: griddepcontrol.launch_dependents is issued at once and the next kernel
//     streams its first stages while this one computes; its consumers wait in
//     griddepcontrol.wait for the activations.
//   * Split-K is ordered and stays on chip: the CTAs that split one column tile form a
//     thread-block cluster and rank 0 adds their partial sums in rank order out of
//     distributed shared memory, so results are bit-identical run to run; the reference's
//     atom.global.add.f32 split-K is not reproduced.  Every mbarrier wait is bounded and
//     reports through a status word instead of hanging.
#include "gemv_core.cuh"

#define GEMV_CONSUMER_WARPS 4
#define GEMV_CONSUMERS (GEMV_CONSUMER_WARPS * 32)

__device__ __forceinline__ void consumer_bar() { asm volatile("bar.sync 1, %0;" ::"n"(GEMV_CONSUMERS) : "memory"); }

// cluster helpers: the CTAs that split one column tile along K form a thread-block cluster and
// combine their partial sums through distributed shared memory
__device__ __forceinline__ uint32_t cluster_ctarank() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ float ld_cluster_f32(const float* local_ptr, uint32_t rank) {
    uint32_t remote; float v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(local_ptr)), "r"(rank));
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
    return v;
}

extern "C" __global__ void __launch_bounds__(GEMV_CONSUMERS + 32, 4) gemv_int4_w256(const __grid_constant__ lb_gemv_params p) {
    extern __shared__ unsigned char smem_raw[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int tile = blockIdx.x, split = blockIdx.y;
    const int n0 = tile * LB_GEMV_TILE_N;
    const int ncols = min(LB_GEMV_TILE_N, p.N - n0);
    const int groups = p.K / LB_GEMV_GROUP;
    const int g0 = split * p.groups_per_split;
    const int g1 = min(groups, g0 + p.groups_per_split);
    const int n_groups = max(0, g1 - g0); // one pipeline stage per group
    const int S = p.stages;

    // shared-memory carve-up; the swizzled boxes need 1024-byte alignment
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    unsigned char* smem = smem_raw + (smem_base - smem_u32(smem_raw));
    __half* sc_s = reinterpret_cast<__half*>(smem + (size_t)S * GEMV_STAGE_BYTES);                     // [groups][256] group scales
    uint32_t* zr_s = reinterpret_cast<uint32_t*>(sc_s + (size_t)p.groups_per_split * LB_GEMV_TILE_N); // [groups][32] zero-point words
    uint32_t* xdig = zr_s + (size_t)p.groups_per_split * (LB_GEMV_TILE_N / 8);                         // digit table of this K slice
    const int dig_words = (digit_row_word(p.groups_per_split * LB_GEMV_ROWS) + 3) & ~3;
    int* xsum = reinterpret_cast<int*>(xdig + dig_words);                 // [groups] integer sum of the group's x
    float* red = reinterpret_cast<float*>(xsum + ((p.groups_per_split + 3) & ~3)); // [256] + 40
    uint64_t* full = reinterpret_cast<uint64_t*>(red + LB_GEMV_TILE_N + 40);
    uint64_t* empty = full + S;
    uint64_t* aux = empty + S; // completion of the scale / zero-point boxes
    __shared__ uint32_t s_bad;

    if (tid == 0) {
        for (int s = 0; s < S; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], GEMV_CONSUMER_WARPS);
        }
        mbar_init(aux, 1);
        s_bad = 0;
        mbar_fence_init();
    }
    __syncthreads();

    if (warp == GEMV_CONSUMER_WARPS) {
        // ---------------- producer: one elected lane streams stages into the ring ----------------
        // Weights never change, so this starts before griddepcontrol.wait.
        if (lane == 0) {
            const uint64_t pol = l2_policy_evict_first();
            // Small requests first: once the bulk stream is queued, any other load waits behind
            // megabytes of weight traffic.  The slice's scales and zero-points are two boxes.
            const uint32_t sc_bytes = (uint32_t)p.groups_per_split * LB_GEMV_TILE_N * 2, zr_bytes = sc_bytes / 4;
            mbar_arrive_expect_tx(aux, sc_bytes + (p.qzeros ? zr_bytes : 0u));
            tma_load_2d(smem_u32(sc_s), p.tmap_sc, n0, g0, aux, pol);
            if (p.qzeros) tma_load_2d(smem_u32(zr_s), p.tmap_zr, n0 >> 3, g0, aux, pol);
            for (int u = 0; u < n_groups; ++u) {
                const int s = u % S;
                if (u >= S && !mbar_wait(&empty[s], ((u / S) - 1) & 1)) {
                    atomicExch(p.status, LB_DEV_TIMEOUT_EMPTY);
                    s_bad = 1;
                    break;
                }
                mbar_arrive_expect_tx(&full[s], GEMV_STAGE_BYTES); // out-of-range parts of the box are zero-filled
                tma_load_stage(smem_base + (uint32_t)s * GEMV_STAGE_BYTES, p.tmap, n0 >> 5, (g0 + u) * LB_GEMV_ROWS, &full[s], pol);
            }
        }
        // consumers wait for every stage, so no copy is in flight past their loop; the warp
        // stays for the cluster barriers below
    }

    const int fg = lane >> 2, ft = lane & 3; // fragment row group / k-slot group of this lane
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    float unit = 1.0f; // value of one integer step of the quantised activations (2^-shift)
    if (warp < GEMV_CONSUMER_WARPS) {
        if (!p.qzeros) // zero-point 8 everywhere
            for (int i = tid; i < n_groups * (LB_GEMV_TILE_N / 8); i += GEMV_CONSUMERS) zr_s[i] = 0x88888888u;
        pdl_wait(); // x (and y for accumulate mode) come from the previous kernel
        const int rows = n_groups * LB_GEMV_ROWS;
        const int row0 = g0 * LB_GEMV_ROWS; // first packed row of this split

        // --- prologue: the activation slice as exact integers -------------------------------
        // X_k = rint(x_k * 2^shift) with |X| < 2^22, split into three signed base-256 digits; the
        // digits are the B operand of the integer MMA (one B column per digit plane).  x_k is
        // fp16, so X_k is EXACT for every element within 2^-11 of the slice maximum and off by at
        // most max|x| * 2^-23 below that.
        float rinv = 1.0f;
        if (p.x_mode == LB_X_F32_RMSNORM) {
            const float4* xv = reinterpret_cast<const float4*>(p.x);
            float ss = 0.f;
            for (int i = tid; i < p.K / 4; i += GEMV_CONSUMERS) {
                float4 v = __ldg(xv + i);
                ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
            }
            ss = warp_sum(ss);
            if (lane == 0) red[warp] = ss;
            consumer_bar();
            float tot = 0.f;
#pragma unroll
            for (int w = 0; w < GEMV_CONSUMER_WARPS; ++w) tot += red[w];
            rinv = rsqrtf(tot / (float)p.K + p.eps);
            consumer_bar();
        }
        float vmax = 0.f;
        for (int rb = 0; rb < rows; rb += GEMV_CONSUMERS) {
            float v[8];
            const int r = rb + tid;
            load_x_row<false>(p, (row0 + r) * 8, r < rows, rinv, v);
#pragma unroll
            for (int j = 0; j < 8; ++j) vmax = fmaxf(vmax, fabsf(v[j]));
            if (r < rows) { // parked as fp16 in the row's own digit slot until the scale is known
                __half2 pk[4] = {__floats2half2_rn(v[0], v[1]), __floats2half2_rn(v[2], v[3]),
                                 __floats2half2_rn(v[4], v[5]), __floats2half2_rn(v[6], v[7])};
                uint32_t* dst = xdig + digit_row_word(r);
                const uint32_t* pw = reinterpret_cast<const uint32_t*>(pk);
                *reinterpret_cast<uint2*>(dst) = make_uint2(pw[0], pw[1]);
                *reinterpret_cast<uint2*>(dst + 2) = make_uint2(pw[2], pw[3]);
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) vmax = fmaxf(vmax, __shfl_xor_sync(0xffffffffu, vmax, o));
        if (lane == 0) red[8 + warp] = vmax;
        consumer_bar();
        vmax = fmaxf(fmaxf(red[8], red[9]), fmaxf(red[10], red[11]));
        // shift so that max|x| * 2^shift lies in [2^21, 2^22); all-zero or non-finite slices use shift 0
        int shift = 0;
        if (vmax > 0.f && vmax < 3.0e38f) shift = 21 - (int)((__float_as_uint(vmax) >> 23) & 0xffu) + 127;
        const float qscale = __uint_as_float((uint32_t)(127 + shift) << 23); // 2^shift (|shift| < 60 for fp16 data)
        unit = __uint_as_float((uint32_t)(127 - shift) << 23);
        for (int rb = 0; rb < rows; rb += GEMV_CONSUMERS) {
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
            int X[8], rs = 0;
            uint32_t ev[3] = {0u, 0u, 0u}, od[3] = {0u, 0u, 0u};
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                X[j] = __float2int_rn(v[j] * qscale);
                rs += X[j];
                int t = X[j];
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
            for (int o = 8; o > 0; o >>= 1) rs += __shfl_xor_sync(0xffffffffu, rs, o); // the group's 16 rows
            if (live) {
                uint32_t* dst = xdig + digit_row_word(r);
#pragma unroll
                for (int d = 0; d < 3; ++d) *reinterpret_cast<uint2*>(dst + 2 * d) = make_uint2(ev[d], od[d]);
                if ((lane & 15) == 0) xsum[r >> 4] = rs;
                if (p.x_out && tile == 0) {
                    __half2 pl[4] = {__floats2half2_rn(v[0], v[1]), __floats2half2_rn(v[2], v[3]),
                                     __floats2half2_rn(v[4], v[5]), __floats2half2_rn(v[6], v[7])};
                    *reinterpret_cast<uint4*>(p.x_out + (row0 + r) * 8) = *reinterpret_cast<uint4*>(pl);
                }
            }
        }
        consumer_bar();

        // --- main loop: one group (16 packed rows x 256 columns) per stage; a warp takes two
        //     adjacent 32-column boxes.  Box rows are 128 B; the 16-byte chunk c of row r sits at
        //     chunk c ^ (r & 7) (128-byte swizzle).  In step e a lane reads packed row
        //     8*(e>>1) + 2*ft + (e&1), chunk fg: the 8 lanes of a quarter-warp then hit 8 different
        //     chunks (no bank conflict), and all lanes with the same ft share one packed row, as
        //     the MMA k-slots need.  Lanes fg = 0,1,2 supply the three digit planes as B columns.
        if (!mbar_wait(aux, 0)) {
            if (lane == 0) { atomicExch(p.status, LB_DEV_TIMEOUT_FULL); s_bad = 1; }
        }
        const int cbase = warp * 64;                  // this warp's first column inside the tile
        const bool live0 = cbase < ncols, live1 = cbase + 32 < ncols; // N % 32 == 0: a box is all valid or all past N
        // lane ft holds B columns 2ft, 2ft+1 of the result: ft=0 digits 0 and 1, ft=1 digit 2
        const float lane_mul = ft == 0 ? 1.0f : (ft == 1 ? 65536.0f : 0.0f);
        const bool has_digits = fg < 3;
        for (int u = 0; u < n_groups; ++u) {
            const int s = u % S;
            uint2 sraw[2];
            uint32_t zw[2];
            sraw[0] = *reinterpret_cast<const uint2*>(sc_s + u * LB_GEMV_TILE_N + cbase + fg * 4);
            sraw[1] = *reinterpret_cast<const uint2*>(sc_s + u * LB_GEMV_TILE_N + cbase + 32 + fg * 4);
            zw[0] = zr_s[u * (LB_GEMV_TILE_N / 8) + ((cbase + fg * 4) >> 3)];
            zw[1] = zr_s[u * (LB_GEMV_TILE_N / 8) + ((cbase + 32 + fg * 4) >> 3)];
            if (!mbar_wait(&full[s], (u / S) & 1)) {
                if (lane == 0) { atomicExch(p.status, LB_DEV_TIMEOUT_FULL); s_bad = 1; }
                break;
            }
            int d[2][2][4]; // [box][column pair][fragment]
#pragma unroll
            for (int i = 0; i < 16; ++i) (&d[0][0][0])[i] = 0;
            if (live0) {
                const unsigned char* box = smem + (size_t)s * GEMV_STAGE_BYTES + (warp * 2) * GEMV_BOX_BYTES;
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int r = 8 * (e >> 1) + 2 * ft + (e & 1);
                    uint2 xb = make_uint2(0u, 0u);
                    if (has_digits) xb = *reinterpret_cast<const uint2*>(xdig + digit_row_word(u * LB_GEMV_ROWS + r) + 2 * fg);
                    const uint32_t off = r * 128 + ((fg ^ (r & 7)) << 4);
                    const uint4 w0 = *reinterpret_cast<const uint4*>(box + off);
                    imma_words(d[0][0], w0.x, w0.y, xb);
                    imma_words(d[0][1], w0.z, w0.w, xb);
                    if (live1) {
                        const uint4 w1 = *reinterpret_cast<const uint4*>(box + GEMV_BOX_BYTES + off);
                        imma_words(d[1][0], w1.x, w1.y, xb);
                        imma_words(d[1][1], w1.z, w1.w, xb);
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[s]); // this warp is done with the stage
            // per column: (sum q X) - z * (sum X), times the fp16 group scale.  Fragment element 0/2
            // is B column 2ft (row g / g+8), element 1/3 is B column 2ft+1: digit d and d+1.
            const float xs_f = ft == 0 ? (float)xsum[u] : 0.f;
#pragma unroll
            for (int b = 0; b < 2; ++b) {
                const float2 s01 = __half22float2(*reinterpret_cast<const __half2*>(&sraw[b].x));
                const float2 s23 = __half22float2(*reinterpret_cast<const __half2*>(&sraw[b].y));
                const uint32_t z = zw[b] >> ((fg & 1) * 16);
                const float sc[4] = {s01.x, s01.y, s23.x, s23.y};
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const int* f = d[b][c >> 1];
                    const int comb = f[(c & 1) * 2] + (f[(c & 1) * 2 + 1] << 8);
                    const float zf = __uint_as_float(0x4B000000u | ((z >> (4 * c)) & 0xFu)) - 8388608.0f;
                    acc[b * 4 + c] = fmaf(sc[c], fmaf(-zf, xs_f, (float)comb * lane_mul), acc[b * 4 + c]);
                }
            }
        }
        pdl_launch_dependents(); // the next kernel may become resident while this one reduces
        // add the digit planes held by the four ft lanes (fixed order), scale back to x units
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            float a = acc[i];
            a += __shfl_xor_sync(0xffffffffu, a, 1);
            a += __shfl_xor_sync(0xffffffffu, a, 2);
            acc[i] = a * unit;
        }
        if (ft == 0) {
            *reinterpret_cast<float4*>(red + cbase + fg * 4) = make_float4(acc[0], acc[1], acc[2], acc[3]);
            *reinterpret_cast<float4*>(red + cbase + 32 + fg * 4) = make_float4(acc[4], acc[5], acc[6], acc[7]);
        }
    } // consumer warps

    // --- ordered split-K: the ksplit CTAs of a tile are one cluster; rank 0 adds the partial sums
    //     of ranks 0,1,2,... in that order out of their shared memory ---
    float v0 = 0.f, v1 = 0.f; // columns tid and tid + 128 (the block has 160 threads, the tile 256 columns)
    const bool owner = tid < 128;
    if (p.ksplit > 1) {
        cluster_sync_all();
        if (cluster_ctarank() == 0 && owner)
            for (uint32_t r = 0; r < (uint32_t)p.ksplit; ++r) {
                v0 += ld_cluster_f32(red + tid, r);
                v1 += ld_cluster_f32(red + 128 + tid, r);
            }
        cluster_sync_all(); // nobody leaves while rank 0 is still reading its shared memory
        if (cluster_ctarank() != 0) return;
    } else {
        __syncthreads();
        if (owner) { v0 = red[tid]; v1 = red[128 + tid]; }
    }

    // --- epilogue ---
    if (s_bad) return;
    if (p.y_mode == LB_Y_SWIGLU_F16) {
        // columns come in interleaved 64-wide (gate, up) blocks: [0,64) gate, [64,128) up, ...
        __syncthreads();
        if (owner) { red[tid] = v0; red[128 + tid] = v1; }
        __syncthreads();
        if (owner && tid < ncols / 2) {
            const int blk = tid >> 6, i = tid & 63;
            const float gate = red[blk * 128 + i], up = red[blk * 128 + 64 + i];
            reinterpret_cast<__half*>(p.y)[n0 / 2 + tid] = __float2half_rn(siluf_dev(gate) * up);
        }
        return;
    }
    if (owner) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int c = tid + 128 * h;
            const float v = h ? v1 : v0;
            if (c < ncols) {
                const int n = n0 + c;
                if (p.y_mode == LB_Y_F16) reinterpret_cast<__half*>(p.y)[n] = __float2half_rn(v);
                else if (p.y_mode == LB_Y_F32) reinterpret_cast<float*>(p.y)[n] = v;
                else reinterpret_cast<float*>(p.y)[n] += v;
            }
        }
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
    float best_v = -INFINITY;
    int best_i = 0x7fffffff;
    for (int n = blockIdx.x * nwarps + warp; n < p.N; n += gridDim.x * nwarps) {
        const uint4* wr = reinterpret_cast<const uint4*>(p.w + (size_t)n * p.K);
        float a0 = 0.f, a1 = 0.f;
#pragma unroll 5
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
        if (t > best_v || (t == best_v && n < best_i)) { best_v = t; best_i = n; }
    }
    if (p.part_val) { // this CTA's candidate for the arg-max: greater value, smaller row on ties
        __syncthreads();
        int* ri = reinterpret_cast<int*>(red + 16);
        if (lane == 0) { red[warp] = best_v; ri[warp] = best_i; }
        __syncthreads();
        if (tid == 0) {
            for (int w = 1; w < nwarps; ++w)
                if (red[w] > best_v || (red[w] == best_v && ri[w] < best_i)) { best_v = red[w]; best_i = ri[w]; }
            p.part_val[blockIdx.x] = best_v;
            p.part_idx[blockIdx.x] = best_i;
        }
    }
}

// ---------------------------------------------------------------------------
// The same dense bf16 [N,K] x vector product, streamed: one CTA per SM, every warp requests whole
// rows (K * 2 bytes, contiguous) with 1-D bulk copies into its own two ring slots and consumes
// them from shared memory, so the HBM stream does not depend on per-thread loads in flight.
// Row n goes to CTA n % gridDim.x, warp (n / gridDim.x) % 8.  Same prologues, results and arg-max
// candidates as dense_bf16_gemv (one candidate per CTA).  Used for the LM head
// (src/launcher.s:2903-2970) when a row fits a ring slot.
// ---------------------------------------------------------------------------
#define DS_WARPS 8
#define DS_SLOTS 2
extern "C" __global__ void __launch_bounds__(DS_WARPS * 32, 1) dense_bf16_stream(const __grid_constant__ lb_dense_params p) {
    extern __shared__ __align__(16) unsigned char ds_sm[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t row_bytes = (uint32_t)p.K * 2u;
    unsigned char* ring = ds_sm;                                                          // [8 warps][2 slots][row]
    float* xsm = reinterpret_cast<float*>(ds_sm + (size_t)DS_WARPS * DS_SLOTS * row_bytes); // [K] fp32
    float* red = xsm + p.K;                                                               // [40]
    uint64_t* bars = reinterpret_cast<uint64_t*>(red + 40);                               // [8][2]
    if (lane == 0)
        for (int s = 0; s < DS_SLOTS; ++s) mbar_init(&bars[warp * DS_SLOTS + s], 1);
    mbar_fence_init();
    __syncwarp();
    // rows of this warp: n = (warp + 8 m) * G + c; weights are constants: the first requests go out before griddepcontrol.wait
    const int G = gridDim.x, c = blockIdx.x;
    const int my_rows = p.N > c ? ((p.N - c + G - 1) / G - warp + DS_WARPS - 1) / DS_WARPS : 0; // rows (p.N - c)/G of the CTA, every 8th
    const uint64_t pol = l2_policy_evict_first();
    auto request = [&](int m) {
        if (lane == 0) {
            const size_t n = (size_t)(warp + DS_WARPS * m) * G + c;
            uint64_t* bar = &bars[warp * DS_SLOTS + (m % DS_SLOTS)];
            mbar_arrive_expect_tx(bar, row_bytes);
            bulk_g2s(ring + ((size_t)warp * DS_SLOTS + (m % DS_SLOTS)) * row_bytes, p.w + n * p.K, row_bytes, bar, pol);
        }
    };
    for (int m = 0; m < DS_SLOTS && m < my_rows; ++m) request(m);

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

    float best_v = -INFINITY;
    int best_i = 0x7fffffff;
    for (int m = 0; m < my_rows; ++m) {
        const int slot = m % DS_SLOTS;
        if (!__all_sync(0xffffffffu, mbar_wait(&bars[warp * DS_SLOTS + slot], (m / DS_SLOTS) & 1))) { // bounded: the rows left keep y unset
            if (lane == 0 && p.status) atomicExch(p.status, LB_DEV_TIMEOUT_FULL);
            break;
        }
        const uint4* wr = reinterpret_cast<const uint4*>(ring + ((size_t)warp * DS_SLOTS + slot) * row_bytes);
        float a0 = 0.f, a1 = 0.f;
#pragma unroll 4
        for (int i = lane; i < p.K / 8; i += 32) { // same order of additions as dense_bf16_gemv
            const uint4 w = wr[i];
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
        __syncwarp(); // every lane has its words in registers (the sums depend on them): the slot can be refilled
        if (m + DS_SLOTS < my_rows) request(m + DS_SLOTS);
        const float t = warp_sum(a0 + a1);
        const int n = (warp + DS_WARPS * m) * G + c;
        if (lane == 0) p.y[n] = t;
        if (t > best_v || (t == best_v && n < best_i)) { best_v = t; best_i = n; }
    }
    if (p.part_val) { // this CTA's candidate for the arg-max: greater value, smaller row on ties
        __syncthreads();
        int* ri = reinterpret_cast<int*>(red + 16);
        if (lane == 0) { red[warp] = best_v; ri[warp] = best_i; }
        __syncthreads();
        if (tid == 0) {
            for (int w = 1; w < DS_WARPS; ++w)
                if (red[w] > best_v || (red[w] == best_v && ri[w] < best_i)) { best_v = red[w]; best_i = ri[w]; }
            p.part_val[blockIdx.x] = best_v;
            p.part_idx[blockIdx.x] = best_i;
        }
    }
}
