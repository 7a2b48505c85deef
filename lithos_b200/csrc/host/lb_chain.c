/* Host side of the persistent GEMV chain (kernels/chain.cu): checks, the per-GEMV tensor maps and
 * the single launch.  The reference issues one launch_gemv per projection
 * (src/launcher.s:1226-1535); a chain replaces a run of them. */
#include "lb_internal.h"
#include "../kernels/params.h"

_Static_assert(sizeof(lb_chain_params) <= 4096, "kernel parameter block limit");
_Static_assert(LB_GEMV_CHAIN_MAX == LB_CHAIN_MAX_OPS, "public and kernel limits agree");

/* ring depth: what one SM's shared memory holds next to the activation table, minus room for a small
 * CTA of the neighbouring kernel (programmatic dependent launch lets it become resident early) */
static int chain_stages(const lb_ctx* c, unsigned* smem_out) {
    const size_t dig_words = (size_t)((6 * LB_CHAIN_XCAP * LB_GEMV_ROWS + 2 * (LB_CHAIN_XCAP * LB_GEMV_ROWS >> 2) + 3) & ~3);
    const size_t fixed = 1024 + dig_words * 4 + 64;
    const size_t budget = (size_t)c->max_smem_optin - 4096 /* static shared memory of the kernel */ - (size_t)c->chain_reserve;
    int st = budget > fixed ? (int)((budget - fixed) / (LB_CHAIN_STAGE_STRIDE + 16)) : 0;
    if (st > 12) st = 12;
    if (smem_out) *smem_out = (unsigned)(fixed + (size_t)st * (LB_CHAIN_STAGE_STRIDE + 16));
    return st;
}

static int chain_check_shape(lb_ctx* c, int K, int N) {
    if (K <= 0 || N <= 0 || K % LB_GEMV_GROUP != 0 || N % 32 != 0)
        return lb_fail(c, LB_ERR_INVALID, "GEMV chain needs K %% 128 == 0 and N %% 32 == 0 (K=%d, N=%d)", K, N);
    const int kg = K / LB_GEMV_GROUP, tiles = (N + LB_GEMV_TILE_N - 1) / LB_GEMV_TILE_N;
    const long long units = (long long)kg * tiles;
    const int G = c->sm_count;
    if (tiles > LB_CHAIN_MAX_TILES) return lb_fail(c, LB_ERR_INVALID, "GEMV chain: N=%d has more than %d column tiles", N, LB_CHAIN_MAX_TILES);
    if (units < G) return lb_fail(c, LB_ERR_INVALID, "GEMV chain: K=%d N=%d is %lld units, fewer than the %d SMs", K, N, units, G);
    /* K-groups one CTA meets: all of them when its range spans a tile, else its range length */
    const long long per_cta = (units + G - 1) / G;
    const long long window = per_cta >= kg ? kg : per_cta;
    if (window > LB_CHAIN_XCAP)
        return lb_fail(c, LB_ERR_INVALID, "GEMV chain: K=%d N=%d needs %lld K-groups of activations per CTA (max %d)", K, N,
                       window, LB_CHAIN_XCAP);
    return LB_OK;
}

LB_API int lb_gemv_chain_supports(lb_ctx* c, int K, int N) {
    if (!c) return LB_ERR_INVALID;
    return chain_check_shape(c, K, N);
}

LB_API int lb_gemv_chain(lb_ctx* c, const lb_gemv_op* ops, int n_ops) {
    if (!c || !ops) return LB_ERR_INVALID;
    if (n_ops < 1 || n_ops > LB_CHAIN_MAX_OPS) return lb_fail(c, LB_ERR_INVALID, "GEMV chain: %d entries (1..%d)", n_ops, LB_CHAIN_MAX_OPS);
    lb_chain_params p;
    memset(&p, 0, sizeof p);
    for (int i = 0; i < n_ops; i++) {
        const lb_gemv_op* o = &ops[i];
        if (!o->qweight || !o->scales || !o->x || !o->y) return lb_fail(c, LB_ERR_INVALID, "GEMV chain[%d]: NULL operand", i);
        if (o->x_mode < LB_X_F16 || o->x_mode > LB_X_F32_HEADNORM_SILU || o->y_mode < LB_Y_F16 || o->y_mode > LB_Y_SWIGLU_F16)
            return lb_fail(c, LB_ERR_INVALID, "GEMV chain[%d]: unknown x_mode/y_mode %d/%d", i, o->x_mode, o->y_mode);
        if ((o->x_mode == LB_X_F32_RMSNORM && !o->aux0) || (o->x_mode == LB_X_F32_HEADNORM_SILU && (!o->aux0 || !o->aux1)))
            return lb_fail(c, LB_ERR_INVALID, "GEMV chain[%d]: norm prologue without its weight/gate operand", i);
        if (o->y_mode == LB_Y_SWIGLU_F16 && o->N % 128 != 0)
            return lb_fail(c, LB_ERR_INVALID, "GEMV chain[%d]: SwiGLU epilogue needs N %% 128 == 0 (N=%d)", i, o->N);
        if (((o->qweight | o->scales | o->qzeros | o->x | o->y | o->aux0 | o->aux1 | o->x_out) & 15ull) != 0)
            return lb_fail(c, LB_ERR_INVALID, "GEMV chain[%d]: operands must be 16-byte aligned", i);
        LB_TRY(chain_check_shape(c, o->K, o->N));
        lb_chain_op* d = &p.op[i];
        LB_TRY(lb_gemv_tensor_maps(c, o->qweight, o->scales, o->qzeros, o->K, o->N, 1, d->tmap, d->tmap_sc, d->tmap_zr));
        d->x = (const void*)o->x; d->y = (void*)o->y;
        d->aux0 = (const void*)o->aux0; d->aux1 = (const void*)o->aux1;
        d->x_out = (uint16_t*)o->x_out;
        d->K = o->K; d->N = o->N;
        d->kg = o->K / LB_GEMV_GROUP;
        d->units = d->kg * ((o->N + LB_GEMV_TILE_N - 1) / LB_GEMV_TILE_N);
        d->x_mode = o->x_mode; d->y_mode = o->y_mode;
        d->has_zeros = o->qzeros ? 1 : 0;
        d->eps = o->eps;
    }
    unsigned smem = 0;
    p.stages = chain_stages(c, &smem);
    if (p.stages < 2) return lb_fail(c, LB_ERR_INVALID, "GEMV chain: shared memory holds %d stages", p.stages);
    p.n_ops = n_ops;
    p.trigger_op = n_ops - 1;
    p.status = (uint32_t*)c->dev_status;
    p.tile_count = (uint32_t*)c->gemv_counters;               /* words [0, LB_CHAIN_MAX_TILES) */
    p.sync = (uint32_t*)c->gemv_counters + LB_CHAIN_MAX_TILES; /* two words */
    p.partial = (float*)c->gemv_partial;
    void* params[] = {&p};
    return lb_launch(c, LBK_gemv_chain, (unsigned)c->sm_count, 1, 1, LB_CHAIN_THREADS, smem, params, 1);
}
