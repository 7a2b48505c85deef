/* Per-kernel launch wrappers: argument checks, launch geometry, parameter
 * blocks.  These are the C counterparts of the reference's launch_* helpers
 * (src/launcher.s:1101-2975), one per kernel family. */
#include "lb_internal.h"
#include "../kernels/params.h"
#include <math.h>

#define GEMV_THREADS LB_GEMV_THREADS

/* Geometry of one int4 GEMV launch.
 *  - grid = (column tiles of 128, ksplit); the ksplit CTAs of a tile form one cluster and add
 *    their partial sums on chip, so ksplit <= 8.
 *  - All CTAs of a launch should be co-resident and carry equal work, so that the HBM pipe and
 *    not a tail of late CTAs ends the kernel: ksplit is chosen so that tiles*ksplit comes close
 *    to (and not above) two CTAs per SM.
 *  - A CTA's shared memory (ring of 16 KB stages + its activation slice) is kept under a quarter
 *    of an SM where possible, so that the CTAs of the NEXT kernel fit beside it and prefetch
 *    their weights while this one computes (programmatic dependent launch). */
typedef struct { int tiles, ksplit, gps, stages; unsigned smem; } gemv_geom;

static int gemv_plan(lb_ctx* c, int K, int N, gemv_geom* g) {
    if (K <= 0 || N <= 0 || K % LB_GEMV_GROUP != 0 || N % 32 != 0)
        return lb_fail(c, LB_ERR_INVALID, "int4 GEMV needs K %% 128 == 0 and N %% 32 == 0 (K=%d, N=%d)", K, N);
    int groups = K / LB_GEMV_GROUP;
    g->tiles = (N + LB_GEMV_TILE_N - 1) / LB_GEMV_TILE_N;
    int slots = 2 * c->sm_count;
    int ks = slots / g->tiles;
    if (ks < 1) ks = 1;
    if (ks > LB_GEMV_MAX_SPLITS) ks = LB_GEMV_MAX_SPLITS;
    if (ks > groups) ks = groups;
    g->gps = (groups + ks - 1) / ks;
    g->ksplit = (groups + g->gps - 1) / g->gps;
    /* shared memory: 1 KB alignment slack, ring of 16 KB stages (one group each), the digit
     * table of the K slice (26 bytes per packed row), per-group sums, result buffer, mbarriers */
    int rows = g->gps * LB_GEMV_ROWS;
    size_t dig_words = (size_t)((6 * rows + 2 * (rows >> 2) + 3) & ~3);
    size_t fixed = 1024 + dig_words * 4 + (size_t)((g->gps + 3) & ~3) * 4 + (LB_GEMV_TILE_N + 40) * 4 +
                   (size_t)g->gps * (LB_GEMV_TILE_N * 2 + LB_GEMV_TILE_N / 2); /* + group scales and zero-points */
    fixed += 16; /* the scale-box mbarrier */
    size_t per_stage = LB_GEMV_STAGE_BYTES + 16; /* stage + its two mbarriers */
    size_t sm_total = (size_t)c->max_smem_optin + 1024; /* shared memory of one SM */
    int st = 0;
    for (int per_sm = 4; per_sm >= 1 && st < 2; per_sm >>= 1) {
        size_t budget = sm_total / per_sm - 1024;
        if (budget > (size_t)c->max_smem_optin) budget = (size_t)c->max_smem_optin;
        st = budget > fixed ? (int)((budget - fixed) / per_stage) : 0;
    }
    if (st < 1) return lb_fail(c, LB_ERR_INVALID, "int4 GEMV: K slice of %d groups does not fit shared memory", g->gps);
    if (st > 6) st = 6;
    if (st > g->gps) st = g->gps;
    g->stages = st;
    g->smem = (unsigned)((fixed + (size_t)st * per_stage + 127) & ~(size_t)127);
    return LB_OK;
}

/* The three tensor maps of one int4 matrix.
 * qweight is viewed as [N/32 column blocks][K/8 packed rows][32 columns] so that ONE tiled load
 * brings a whole stage: box = 8 column blocks x 16 rows x 32 columns, laid down as eight
 * consecutive 2 KB boxes with the 128-byte swizzle.  Parts of the box past the matrix
 * (ragged last tile, last group) are zero-filled and never used.  Scales fp16 [K/128, N] and
 * zero-points u32 [K/128, N/8] come as boxes of box_groups rows x one column tile. */
static int lb_gemv_tensor_maps(lb_ctx* c, uint64_t qweight, uint64_t scales, uint64_t qzeros, int K, int N, int box_groups,
                        unsigned char* tm_w, unsigned char* tm_sc, unsigned char* tm_zr) {
    CUtensorMap tm;
    cuuint64_t dims[3] = {32, (cuuint64_t)(K / 8), (cuuint64_t)(N / 32)};
    cuuint64_t strides[2] = {(cuuint64_t)N * 4, 128};
    cuuint32_t box[3] = {32, LB_GEMV_ROWS, LB_GEMV_TILE_N / 32};
    cuuint32_t estr[3] = {1, 1, 1};
    LB_CU(c, lb_drv.TensorMapEncodeTiled(&tm, CU_TENSOR_MAP_DATA_TYPE_UINT32, 3, (void*)qweight, dims, strides, box,
                                         estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                         CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE));
    memcpy(tm_w, &tm, sizeof tm);
    cuuint64_t sdims[2] = {(cuuint64_t)N, (cuuint64_t)(K / 128)};
    cuuint64_t sstr[1] = {(cuuint64_t)N * 2};
    cuuint32_t sbox[2] = {LB_GEMV_TILE_N, (cuuint32_t)box_groups};
    LB_CU(c, lb_drv.TensorMapEncodeTiled(&tm, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, (void*)scales, sdims, sstr, sbox, estr,
                                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                                         CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE));
    memcpy(tm_sc, &tm, sizeof tm);
    if (qzeros) {
        cuuint64_t zdims[2] = {(cuuint64_t)(N / 8), (cuuint64_t)(K / 128)};
        cuuint64_t zstr[1] = {(cuuint64_t)(N / 8) * 4};
        cuuint32_t zbox[2] = {LB_GEMV_TILE_N / 8, (cuuint32_t)box_groups};
        LB_CU(c, lb_drv.TensorMapEncodeTiled(&tm, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, (void*)qzeros, zdims, zstr, zbox,
                                             estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                                             CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE));
        memcpy(tm_zr, &tm, sizeof tm);
    }
    return LB_OK;
}

LB_API int lb_gemv_int4_fused(lb_ctx* c, uint64_t qweight, uint64_t scales, uint64_t qzeros, uint64_t x, uint64_t y,
                              int K, int N, int x_mode, int y_mode, uint64_t aux0, uint64_t aux1, uint64_t x_out,
                              float eps) {
    if (!c) return LB_ERR_INVALID;
    if (!qweight || !scales || !x || !y) return lb_fail(c, LB_ERR_INVALID, "int4 GEMV: NULL operand");
    if (x_mode < LB_X_F16 || x_mode > LB_X_F32_HEADNORM_SILU || y_mode < LB_Y_F16 || y_mode > LB_Y_SWIGLU_F16)
        return lb_fail(c, LB_ERR_INVALID, "int4 GEMV: unknown x_mode/y_mode %d/%d", x_mode, y_mode);
    if ((x_mode == LB_X_F32_RMSNORM && !aux0) || (x_mode == LB_X_F32_HEADNORM_SILU && (!aux0 || !aux1)))
        return lb_fail(c, LB_ERR_INVALID, "int4 GEMV: norm prologue without its weight/gate operand");
    if (y_mode == LB_Y_SWIGLU_F16 && N % 128 != 0)
        return lb_fail(c, LB_ERR_INVALID, "int4 GEMV: SwiGLU epilogue needs N %% 128 == 0 (N=%d)", N);
    if (((qweight | scales | qzeros | x | y | aux0 | aux1 | x_out) & 15ull) != 0)
        return lb_fail(c, LB_ERR_INVALID, "int4 GEMV: operands must be 16-byte aligned");
    gemv_geom g;
    LB_TRY(gemv_plan(c, K, N, &g));
    lb_gemv_params p;
    memset(&p, 0, sizeof p);
    p.qweight = (const uint32_t*)qweight;
    p.scales = (const uint16_t*)scales;
    p.qzeros = (const uint32_t*)qzeros;
    p.x = (const void*)x;
    p.y = (void*)y;
    p.aux0 = (const void*)aux0;
    p.aux1 = (const void*)aux1;
    p.x_out = (uint16_t*)x_out;
    p.status = (uint32_t*)c->dev_status;
    p.K = K; p.N = N;
    p.ksplit = g.ksplit;
    p.groups_per_split = g.gps;
    p.x_mode = x_mode; p.y_mode = y_mode;
    p.eps = eps;
    p.stages = g.stages;
    LB_TRY(lb_gemv_tensor_maps(c, qweight, scales, qzeros, K, N, g.gps, p.tmap, p.tmap_sc, p.tmap_zr));
    void* params[] = {&p};
    return lb_launch_cluster(c, LBK_gemv_int4_w256, (unsigned)g.tiles, (unsigned)g.ksplit, 1, GEMV_THREADS, g.smem, params, 1,
                             (unsigned)g.ksplit);
}

LB_API int lb_gemv_int4(lb_ctx* c, uint64_t qweight, uint64_t scales, uint64_t qzeros, uint64_t x, uint64_t y, int K,
                        int N, int flags) {
    if (!c) return LB_ERR_INVALID;
    int x_mode = (flags & LB_GEMV_X_F32) ? LB_X_F32 : LB_X_F16;
    int y_mode = (flags & LB_GEMV_Y_SWIGLU) ? LB_Y_SWIGLU_F16
                 : (flags & LB_GEMV_Y_ACCUM) ? LB_Y_F32_ACCUM
                 : (flags & LB_GEMV_Y_F32)   ? LB_Y_F32
                                             : LB_Y_F16;
    /* a strip-packed copy of this matrix exists (lb_gemv_pack): one CTA per SM streams whole columns, no split-K, no cluster */
    const uint64_t packed = lb_packed_lookup(c, qweight, K, N, y_mode == LB_Y_SWIGLU_F16);
    if (packed) {
        lb_gemv_op o;
        memset(&o, 0, sizeof o);
        o.packed = packed;
        o.x = x; o.y = y; o.K = K; o.N = N; o.x_mode = x_mode; o.y_mode = y_mode; o.eps = 1e-6f;
        return lb_gemv_chain(c, &o, 1);
    }
    return lb_gemv_int4_fused(c, qweight, scales, qzeros, x, y, K, N, x_mode, y_mode, 0, 0, 0, 1e-6f);
}

/* Host-buffer entry: the reference-facing call a launcher without device
 * buffers of its own would make.  Device copies of the weights are cached on
 * the context between calls. */
static struct {
    lb_ctx* owner;
    const void *hq, *hs, *hz;
    int K, N;
    CUdeviceptr dq, ds, dz, dx, dy;
} g_host_cache;

static void host_cache_drop(lb_ctx* c) {
    if (g_host_cache.owner != c) return;
    if (g_host_cache.dq) lb_drv.MemFree(g_host_cache.dq);
    if (g_host_cache.ds) lb_drv.MemFree(g_host_cache.ds);
    if (g_host_cache.dz) lb_drv.MemFree(g_host_cache.dz);
    if (g_host_cache.dx) lb_drv.MemFree(g_host_cache.dx);
    if (g_host_cache.dy) lb_drv.MemFree(g_host_cache.dy);
    memset(&g_host_cache, 0, sizeof g_host_cache);
}

void lb_ops_release(lb_ctx* c) { host_cache_drop(c); }

LB_API int lb_gemv_int4_host(lb_ctx* c, const uint32_t* qweight, const uint16_t* scales, const uint32_t* qzeros,
                             const void* x, void* y, int K, int N, int flags, int weights_resident) {
    if (!c || !qweight || !scales || !x || !y) return lb_fail(c, LB_ERR_INVALID, "lb_gemv_int4_host: NULL operand");
    gemv_geom g;
    LB_TRY(gemv_plan(c, K, N, &g));
    LB_CU(c, lb_drv.CtxSetCurrent(c->cu_ctx));
    size_t qb = (size_t)K / 8 * N * 4, sb = (size_t)K / 128 * N * 2, zb = (size_t)K / 128 * N / 2;
    size_t xb = (size_t)K * ((flags & LB_GEMV_X_F32) ? 4 : 2);
    size_t yb = (size_t)((flags & LB_GEMV_Y_SWIGLU) ? N / 2 : N) *
                ((flags & (LB_GEMV_Y_F32 | LB_GEMV_Y_ACCUM)) && !(flags & LB_GEMV_Y_SWIGLU) ? 4 : 2);
    int hit = weights_resident && g_host_cache.owner == c && g_host_cache.hq == qweight && g_host_cache.hs == scales &&
              g_host_cache.hz == qzeros && g_host_cache.K == K && g_host_cache.N == N;
    if (!hit) {
        host_cache_drop(g_host_cache.owner);
        g_host_cache.owner = c;
        LB_CU(c, lb_drv.MemAlloc(&g_host_cache.dq, qb));
        LB_CU(c, lb_drv.MemAlloc(&g_host_cache.ds, sb));
        if (qzeros) LB_CU(c, lb_drv.MemAlloc(&g_host_cache.dz, zb));
        LB_CU(c, lb_drv.MemAlloc(&g_host_cache.dx, (size_t)K * 4));
        LB_CU(c, lb_drv.MemAlloc(&g_host_cache.dy, (size_t)N * 4));
        LB_CU(c, lb_drv.MemcpyHtoDAsync(g_host_cache.dq, qweight, qb, c->stream));
        LB_CU(c, lb_drv.MemcpyHtoDAsync(g_host_cache.ds, scales, sb, c->stream));
        if (qzeros) LB_CU(c, lb_drv.MemcpyHtoDAsync(g_host_cache.dz, qzeros, zb, c->stream));
        g_host_cache.hq = qweight; g_host_cache.hs = scales; g_host_cache.hz = qzeros;
        g_host_cache.K = K; g_host_cache.N = N;
    }
    LB_CU(c, lb_drv.MemcpyHtoDAsync(g_host_cache.dx, x, xb, c->stream));
    if (flags & LB_GEMV_Y_ACCUM) LB_CU(c, lb_drv.MemcpyHtoDAsync(g_host_cache.dy, y, yb, c->stream));
    LB_TRY(lb_gemv_int4(c, g_host_cache.dq, g_host_cache.ds, g_host_cache.dz, g_host_cache.dx, g_host_cache.dy, K, N,
                        flags));
    LB_CU(c, lb_drv.MemcpyDtoHAsync(y, g_host_cache.dy, yb, c->stream));
    LB_CU(c, lb_drv.StreamSynchronize(c->stream));
    return LB_OK;
}

/* ---- batched int4 projection ---------------------------------------------------------
 * 33..64 tokens (9..64 with LB_GEMM_TCGEN05): gemm_int4_tc (tcgen05, one CTA per SM: 128 columns x a K slice);
 * otherwise, or with LB_GEMM_MMA_SYNC, the mma.sync kernels (two CTAs per SM): the faster one at each size
 * as measured (bench.py --workload batched).  The K slices of a column block are the CTAs
 * of one cluster (<= 8); the slice count fills the SMs without starting a second wave and leaves
 * every slice at least four K-groups. */
LB_API int lb_gemm_int4(lb_ctx* c, uint64_t qweight, uint64_t scales, uint64_t qzeros, uint64_t x, uint64_t y, int K, int N,
                        int B, int flags) {
    if (!c || !qweight || !scales || !x || !y || K <= 0 || N <= 0 || K % 128 || N % 16 || B < 1 || B > LB_GEMM_MAX_BATCH ||
        (flags & ~(LB_GEMV_Y_F32 | LB_GEMM_MMA_SYNC | LB_GEMM_TCGEN05)) ||
        ((flags & LB_GEMM_MMA_SYNC) && (flags & LB_GEMM_TCGEN05)) || ((flags & LB_GEMM_TCGEN05) && B <= 8) ||
        ((flags & LB_GEMM_MMA_SYNC) && B > 64))
        return lb_fail(c, LB_ERR_INVALID, "lb_gemm_int4: bad argument (K %% 128, N %% 16, 1 <= B <= %d, flags LB_GEMV_Y_F32, LB_GEMM_MMA_SYNC (up to 64 tokens) or LB_GEMM_TCGEN05 (9 tokens or more))",
                       LB_GEMM_MAX_BATCH);
    lb_bgemm_params p;
    memset(&p, 0, sizeof p);
    p.qweight = (const uint32_t*)qweight; p.scales = (const uint16_t*)scales; p.qzeros = (const uint32_t*)qzeros;
    p.x = (const uint16_t*)x; p.y = (void*)y;
    p.K = K; p.N = N; p.B = B; p.y_f32 = (flags & LB_GEMV_Y_F32) != 0;
    p.status = (uint32_t*)c->dev_status;
    /* one token: the GEMV kernel (TMA-streamed, integer tensor-core products) is the faster path, with the same result type */
    if (B == 1 && !(flags & LB_GEMM_MMA_SYNC) && N % 32 == 0 && ((qweight | scales | qzeros | x | y) & 15ull) == 0)
        if (lb_gemv_int4(c, qweight, scales, qzeros, x, y, K, N, flags & LB_GEMV_Y_F32) == LB_OK) return LB_OK; /* else: the batched kernel */
    const int blocks = (N + 127) / 128, groups = K / 128;
    void* params[] = {&p};
    if ((B > 32 && !(flags & LB_GEMM_MMA_SYNC)) || (flags & LB_GEMM_TCGEN05)) {
        const int nt = B > 128 ? 256 : B > 64 ? 128 : B > 32 ? 64 : B > 16 ? 32 : 16;
        const int ta = nt > 128 || getenv("LB_GEMM_SMEM_A") == NULL; /* weights through tensor memory (default), or the shared-memory operand tiles for comparison (up to 128 tokens) */
        unsigned smem = ta ? (unsigned)((nt > 128 ? 3 : nt > 64 ? 6 : nt > 32 ? 12 : 16) * nt * 256) /* 3..16 activation stages */
                           : (unsigned)(4 * 32768 + (nt > 64 ? 3 : nt > 32 ? 5 : nt > 16 ? 10 : 16) * nt * 256); /* four weight stages + 3..16 activation stages */
        if (smem < (unsigned)nt * 132u * 4u) smem = (unsigned)nt * 132u * 4u; /* the epilogue's partial tile [nt][132] fp32 lies over the stages */
        if (x & 15) return lb_fail(c, LB_ERR_INVALID, "lb_gemm_int4: x must be 16-byte aligned");
        CUtensorMap tm; /* X [B, K] fp16, box = 64 k (128 bytes) x NT tokens, laid down with the 128-byte swizzle */
        cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)B};
        cuuint64_t strides[1] = {(cuuint64_t)K * 2};
        cuuint32_t box[2] = {64, (cuuint32_t)nt};
        cuuint32_t estr[2] = {1, 1};
        LB_CU(c, lb_drv.TensorMapEncodeTiled(&tm, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, (void*)x, dims, strides, box, estr,
                                             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                             CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE));
        memcpy(p.tmap_x, &tm, sizeof tm);
        int ksplit = c->sm_count / blocks;
        if (ksplit > 8) ksplit = 8;
        while (ksplit > 1 && groups / ksplit < 4) ksplit--;
        if (ksplit < 1) ksplit = 1;
        return lb_launch_cluster(c, ta ? (nt > 128 ? LBK_gemm_int4_tc_ta_g1 : LBK_gemm_int4_tc_ta) : nt > 64 ? LBK_gemm_int4_tc_g1 : LBK_gemm_int4_tc, (unsigned)blocks, (unsigned)ksplit, 1, 576, smem, params, 1, (unsigned)ksplit);
    }
    const int rows = B > 32 ? 64 : B > 16 ? 32 : B > 8 ? 16 : 8; /* token rows the CTA stages */
    const int kernel = B > 32 ? LBK_gemm_int4_mma_b64 : B > 16 ? LBK_gemm_int4_mma_b32 : B > 8 ? LBK_gemm_int4_mma_b16 : LBK_gemm_int4_mma_b8;
    const unsigned smem = (unsigned)((B > 16 ? 3 : 4) * rows * 320); /* activation ring (the partial tile reuses it) */
    int ksplit = 1;
    while (ksplit < 8 && blocks * ksplit < c->sm_count * 3 / 2 && groups / (ksplit * 2) >= 4) ksplit *= 2;
    return lb_launch_cluster(c, kernel, (unsigned)blocks, (unsigned)ksplit, 1, 256, smem, params, 1, (unsigned)ksplit);
}

LB_API int lb_gptq_dequant(lb_ctx* c, uint64_t qweight, uint64_t scales, uint64_t qzeros, uint64_t w_out, int K, int N) {
    if (!c || !qweight || !scales || !w_out || K % 128 || N % 8) return lb_fail(c, LB_ERR_INVALID, "lb_gptq_dequant: bad argument");
    void* params[] = {&qweight, &scales, &qzeros, &w_out, &K, &N};
    return lb_launch(c, LBK_gptq_dequant_f32, (unsigned)((N + 255) / 256), (unsigned)(K / 8), 1, 256, 0, params, 0);
}

LB_API int lb_gptq_unpack(lb_ctx* c, uint64_t qweight, uint64_t q_out, int K, int N) {
    if (!c || !qweight || !q_out || K % 8) return lb_fail(c, LB_ERR_INVALID, "lb_gptq_unpack: bad argument");
    void* params[] = {&qweight, &q_out, &K, &N};
    return lb_launch(c, LBK_gptq_unpack_u8, (unsigned)((N + 255) / 256), (unsigned)(K / 8), 1, 256, 0, params, 0);
}

/* shared memory of dense_bf16_stream: 8 warps x 2 ring slots of one row, the fp32 activations, reduction scratch, mbarriers */
static size_t dense_stream_smem(int K) { return (size_t)8 * 2 * K * 2 + (size_t)K * 4 + 40 * 4 + 16 * 8; }
static int dense_streams(const lb_ctx* c, int N, int K) {
    return K % 8 == 0 && N >= 8 * c->sm_count &&
           dense_stream_smem(K) <= (size_t)c->max_smem_optin - (size_t)((c->fn_static_smem[LBK_dense_bf16_stream] + 1023) & ~1023);
}

/* CTAs of the dense GEMV = arg-max candidates it leaves */
int lb_dense_ctas(lb_ctx* c, int N, int K) {
    if (dense_streams(c, N, K)) return c->sm_count; /* one CTA per SM, rows streamed through shared memory */
    int ctas = (N + 7) / 8, cap = c->sm_count * 8;  /* each CTA strides over rows, 8 warps = 8 rows at a time */
    return ctas > cap ? cap : ctas;
}

int lb_dense_launch(lb_ctx* c, uint64_t w, uint64_t x, uint64_t y, int N, int K, int x_mode, uint64_t norm_w, float eps,
                    uint64_t part_val, uint64_t part_idx) {
    if (!c || !w || !x || !y || K % 8 || N <= 0) return lb_fail(c, LB_ERR_INVALID, "dense bf16 GEMV: bad argument");
    lb_dense_params p;
    memset(&p, 0, sizeof p);
    p.w = (const uint16_t*)w; p.x = (const void*)x; p.y = (float*)y; p.norm_w = (const void*)norm_w;
    p.N = N; p.K = K; p.x_mode = x_mode; p.eps = eps;
    p.part_val = (float*)part_val; p.part_idx = (int32_t*)part_idx;
    p.status = (uint32_t*)c->dev_status;
    int ctas = lb_dense_ctas(c, N, K);
    void* params[] = {&p};
    if (dense_streams(c, N, K))
        return lb_launch(c, LBK_dense_bf16_stream, (unsigned)ctas, 1, 1, 256, (unsigned)dense_stream_smem(K), params, 1);
    return lb_launch(c, LBK_dense_bf16_gemv, (unsigned)ctas, 1, 1, 256, (unsigned)(K * 4 + 256), params, 1);
}

LB_API int lb_dense_bf16_gemv(lb_ctx* c, uint64_t w, uint64_t x, uint64_t y, int N, int K, int x_is_f32) {
    return lb_dense_launch(c, w, x, y, N, K, x_is_f32 ? LB_X_F32 : LB_X_F16, 0, 1e-6f, 0, 0);
}

LB_API int lb_deltanet_step(lb_ctx* c, uint64_t state, uint64_t q, uint64_t k, uint64_t v, uint64_t z, uint64_t g,
                            uint64_t beta, uint64_t out, int HV, int HK, int n_steps, int in_is_f32) {
    if (!c || !state || !q || !k || !v || !g || !beta || !out || HV <= 0 || HK <= 0 || HV % HK || n_steps < 1)
        return lb_fail(c, LB_ERR_INVALID, "lb_deltanet_step: bad argument");
    lb_deltanet_params p;
    memset(&p, 0, sizeof p);
    p.state = (float*)state; p.q = (const void*)q; p.k = (const void*)k; p.v = (const void*)v;
    p.z = (const float*)z; p.g = (const float*)g; p.beta = (const float*)beta; p.out = (float*)out;
    p.HV = HV; p.HK = HK;
    void* params[] = {&p, &n_steps};
    return lb_launch(c, in_is_f32 ? LBK_deltanet_step_f32 : LBK_deltanet_step_bf16, (unsigned)HV, 4, 1, 128, 0, params, 1);
}

LB_API int lb_decay_gate(lb_ctx* c, uint64_t a, uint64_t a_log, uint64_t dt_bias, uint64_t b, uint64_t g_out,
                         uint64_t beta_out, int n) {
    if (!c || !a || !a_log || !dt_bias || !g_out || n <= 0) return lb_fail(c, LB_ERR_INVALID, "lb_decay_gate: bad argument");
    lb_decay_params p = {(const float*)a, (const float*)a_log, (const float*)dt_bias, (const float*)b,
                         (float*)g_out, (float*)beta_out, n};
    void* params[] = {&p};
    return lb_launch(c, LBK_decay_gate_beta, (unsigned)((n + 127) / 128), 1, 1, 128, 0, params, 1);
}

/* number of position slices: enough CTAs to fill the GPU twice, at least 64 rows each */
/* attn_decode_mma: a CTA of 8 warps takes a slice of 128 rows (one block of 16 per warp) where the context allows */
int lb_attn_mma_splits(lb_ctx* c, int pos, int HKV) {
    int s = (pos + 127) / 128;
    (void)c; (void)HKV;
    if (s < 1) s = 1;
    if (s > 64) s = 64;
    return s;
}

unsigned lb_attn_mma_smem(int G) {
    return (unsigned)(8 * 2 * 16 * 528 + G * 256 * 4 + 2 * 8 * 528 + 2 * 256 * 4 + 2 * 128 * 4 + 2 * 8 * 8 * 4 + 8 * 8 + 128);
}

LB_API int lb_attention_decode(lb_ctx* c, uint64_t q, uint64_t k_new, uint64_t v_new, uint64_t gate, uint64_t q_norm_w,
                               uint64_t k_norm_w, uint64_t k_cache, uint64_t v_cache, uint64_t out, int pos, int HQ,
                               int HKV, int in_is_f32, int rot_dims, float rope_theta, float eps) {
    if (!c || !q || !k_new || !v_new || !k_cache || !v_cache || !out || pos < 0 || HKV <= 0 || HQ % HKV)
        return lb_fail(c, LB_ERR_INVALID, "lb_attention_decode: bad argument");
    int G = HQ / HKV;
    if (!(G == 1 || G == 2 || G == 3 || G == 4 || G == 6) || HKV > 8)
        return lb_fail(c, LB_ERR_INVALID, "lb_attention_decode: unsupported head ratio %d/%d", HQ, HKV);
    if ((q_norm_w == 0) != (k_norm_w == 0)) return lb_fail(c, LB_ERR_INVALID, "lb_attention_decode: q/k norm weights must come together");
    if (rot_dims < 0 || rot_dims > 128 || rot_dims % 8) return lb_fail(c, LB_ERR_INVALID, "lb_attention_decode: bad rot_dims");
    lb_attn_params p;
    memset(&p, 0, sizeof p);
    p.q = (const void*)q; p.k_new = (const void*)k_new; p.v_new = (const void*)v_new; p.gate = (const void*)gate;
    p.q_norm_w = (const uint16_t*)q_norm_w; p.k_norm_w = (const uint16_t*)k_norm_w;
    p.k_cache = (uint16_t*)k_cache; p.v_cache = (uint16_t*)v_cache; p.out = (float*)out;
    p.scratch = (float*)c->attn_scratch; p.counters = (uint32_t*)(c->gemv_counters + 2048 * 4);
    p.pos = pos; p.HQ = HQ; p.HKV = HKV;
    p.splits = lb_attn_mma_splits(c, pos, HKV);
    p.status = (uint32_t*)c->dev_status;
    p.coop = HKV * p.splits <= c->sm_count;
    p.in_dtype = in_is_f32 ? 1 : 0;
    p.gate_stride = 256; p.q_stride = 256;
    p.rot_dims = rot_dims; p.rope_theta = rope_theta; p.eps = eps;
    for (int i = 0; i < rot_dims / 2; i++) p.rope_freq[i] = exp2(-log2((double)rope_theta) * (double)i / (double)(rot_dims / 2));
    void* params[] = {&p};
    return lb_launch(c, LBK_attn_decode_mma, (unsigned)HKV, (unsigned)p.splits, 1, 256, lb_attn_mma_smem(G), params, 1);
}

LB_API int lb_rmsnorm(lb_ctx* c, uint64_t x, uint64_t res, uint64_t w, uint64_t y, uint64_t sum_out, int rows, int D,
                      float eps, int one_plus_w) {
    if (!c || !x || !w || !y || rows <= 0 || D <= 0) return lb_fail(c, LB_ERR_INVALID, "lb_rmsnorm: bad argument");
    void* params[] = {&x, &res, &w, &y, &sum_out, &D, &eps, &one_plus_w};
    return lb_launch(c, LBK_rmsnorm_f32, (unsigned)rows, 1, 1, 256, 0, params, 1);
}

LB_API int lb_argmax(lb_ctx* c, uint64_t x, int n, uint64_t out_idx) {
    if (!c || !x || !out_idx || n <= 0) return lb_fail(c, LB_ERR_INVALID, "lb_argmax: bad argument");
    uint64_t zero = 0;
    void* params[] = {&x, &n, &out_idx, &zero, &zero, &zero};
    return lb_launch(c, LBK_argmax_f32, 1, 1, 1, 1024, 0, params, 1);
}

LB_API int lb_sample_topk(lb_ctx* c, uint64_t x, int n, float temperature, int top_k, uint64_t seed, uint64_t counter, uint64_t out_idx,
                          uint64_t probs_out, uint64_t idx_out) {
    if (!c || !x || !out_idx || n <= 0 || top_k < 1 || top_k > 64) return lb_fail(c, LB_ERR_INVALID, "lb_sample_topk: bad argument (1 <= top_k <= 64)");
    uint64_t zero = 0;
    void* params[] = {&x, &n, &out_idx, &zero, &zero, &temperature, &top_k, &seed, &counter, &probs_out, &idx_out};
    return lb_launch(c, LBK_topk_sample_f32, 1, 1, 1, 1024, 0, params, 1);
}

LB_API int lb_embed(lb_ctx* c, uint64_t table, uint64_t token, uint64_t out, int D) {
    if (!c || !table || !token || !out || D <= 0) return lb_fail(c, LB_ERR_INVALID, "lb_embed: bad argument");
    void* params[] = {&table, &token, &out, &D};
    return lb_launch(c, LBK_embed_bf16, (unsigned)((D + 1023) / 1024), 1, 1, 256, 0, params, 1);
}
