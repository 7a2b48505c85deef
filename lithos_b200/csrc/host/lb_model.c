/* The decode step of the Qwen3.5-27B-shaped hybrid model: weight table, buffer plan, launch
 * sequence, graph capture.  C re-expression of the reference's host loop
 * (src/launcher.s:685-1092 decode_one_token, :92-141 weight slots, :2981-3136 alloc_buffers,
 * :3284-3683 load_weights) with the layer recipe of compiler/megakernel-link.ls:281-525 and
 * models/families/qwen/qwen3.5/27b/layers/{deltanet,attention}/kernels.ls.
 *
 * Per layer the reference issues 15-17 launches; here it is 5:
 *   DeltaNet layer : [RMSNorm + qkv|z projection]  [a/b proj + conv + SiLU + L2 norms + gates +
 *                    recurrence]  [per-head RMSNorm + silu(z) gate + out projection + residual]
 *   attention layer: [RMSNorm + q|gate|k|v projection]  [q/k norm + RoPE + KV append + split-KV
 *                    attention + sigmoid gate]  [o projection + residual]
 *   MLP            : [RMSNorm + gate|up projection + SwiGLU]  [down projection + residual]
 */
#include "lb_model_priv.h"
#include <math.h>

static void dn_fill_params(const lb_model* m, const layer_t* L, lb_dn_layer_params* p);
extern void lb_prefill_ws_free(lb_model* m);
extern int lb_comm_fill(const lb_comm* m, lb_tp_params* p, int slot, int n);
extern uint64_t lb_comm_slot_ptr(const lb_comm* m, int slot);

extern int lb_chain_fits(lb_ctx* c, const lb_chain_op* ops, int n_ops);
extern int lb_chain_launch(lb_ctx* c, const lb_chain_op* ops, int n_ops);
extern int lb_chain_fill_gemv(lb_ctx* c, lb_chain_op* d, const lb_gemv_op* o, int i);
extern int lb_dense_launch(lb_ctx* c, uint64_t w, uint64_t x, uint64_t y, int N, int K, int x_mode, uint64_t norm_w, float eps,
                           uint64_t part_val, uint64_t part_idx);
extern int lb_dense_ctas(lb_ctx* c, int N, int K);
extern int lb_attn_mma_splits(lb_ctx* c, int pos, int HKV);
extern unsigned lb_attn_mma_smem(int G);

static int is_fa(const lb_model_cfg* c, int l) { return (l % c->fa_period) == c->fa_period - 1; }

static int dalloc(lb_model* m, CUdeviceptr* p, size_t bytes) {
    uint64_t d = 0;
    LB_TRY(lb_malloc(m->c, bytes < 16 ? 16 : bytes, &d));
    *p = (CUdeviceptr)d;
    return LB_OK;
}
static int upload(lb_model* m, CUdeviceptr* p, const void* src, size_t bytes) {
    LB_TRY(dalloc(m, p, bytes));
    LB_CU(m->c, lb_drv.MemcpyHtoDAsync(*p, src, bytes, m->c->stream));
    LB_CU(m->c, lb_drv.StreamSynchronize(m->c->stream)); /* src may be a temporary */
    return LB_OK;
}

LB_API int lb_model_create(lb_ctx* c, const lb_model_cfg* cfg, int tp_rank, int tp_size, lb_model** out) {
    if (!c || !cfg || !out) return LB_ERR_INVALID;
    *out = NULL;
    if (cfg->dn_dim != 128 || cfg->fa_dim != 256 || cfg->group != 128 || cfg->conv_taps != 4)
        return lb_fail(c, LB_ERR_INVALID, "model: kernels are built for dn_dim 128, fa_dim 256, group 128, 4 conv taps");
    if (cfg->hidden % 128 || cfg->inter % 64 || cfg->n_layers < 1 || cfg->fa_period < 1 || cfg->max_ctx < 1 ||
        cfg->dn_v_heads % cfg->dn_k_heads || cfg->fa_q_heads % cfg->fa_kv_heads)
        return lb_fail(c, LB_ERR_INVALID, "model: unsupported shape");
    if (tp_size < 1 || tp_rank < 0 || tp_rank >= tp_size) return lb_fail(c, LB_ERR_INVALID, "model: bad tensor-parallel rank");
    if (cfg->dn_k_heads % tp_size || cfg->dn_v_heads % tp_size || cfg->fa_q_heads % tp_size || cfg->vocab % tp_size ||
        (cfg->inter / 128) % tp_size || (cfg->fa_kv_heads % tp_size && tp_size % cfg->fa_kv_heads))
        return lb_fail(c, LB_ERR_INVALID, "model: heads / intermediate size / vocabulary do not split %d ways", tp_size);
    lb_model* m = (lb_model*)calloc(1, sizeof *m);
    if (!m) return LB_ERR_NOMEM;
    m->c = c; m->cfg = *cfg; m->tp_rank = tp_rank; m->tp_size = tp_size;
    m->use_chain = 1;
    m->HV = cfg->dn_v_heads / tp_size; m->HK = cfg->dn_k_heads / tp_size; m->HQ = cfg->fa_q_heads / tp_size;
    m->HKV = cfg->fa_kv_heads >= tp_size ? cfg->fa_kv_heads / tp_size : 1; /* fewer KV heads than GPUs: replicated */
    m->inter_s = cfg->inter / tp_size;
    m->vocab_s = cfg->vocab / tp_size;
    m->C_s = (2 * m->HK + m->HV) * 128;
    m->L = (layer_t*)calloc((size_t)cfg->n_layers, sizeof(layer_t));
    if (!m->L) { free(m); return LB_ERR_NOMEM; }
    *out = m;
    LB_CU(c, lb_drv.CtxSetCurrent(c->cu_ctx));
    const int H = cfg->hidden;
    int n_in_dn = m->C_s + m->HV * 128, n_in_fa = (2 * m->HQ + 2 * m->HKV) * 256;
    int n_in = n_in_dn > n_in_fa ? n_in_dn : n_in_fa;
    int n_mix = m->HV * 128 > m->HQ * 256 ? m->HV * 128 : m->HQ * 256;
    LB_TRY(dalloc(m, &m->X, (size_t)H * 4));
    LB_TRY(dalloc(m, &m->xn, (size_t)H * 2));
    LB_TRY(dalloc(m, &m->in_out, (size_t)n_in * 4));
    LB_TRY(dalloc(m, &m->mix_out, (size_t)n_mix * 4));
    LB_TRY(dalloc(m, &m->mlp_m, (size_t)m->inter_s * 2));
    LB_TRY(dalloc(m, &m->logits, (size_t)m->vocab_s * 4));
    LB_TRY(dalloc(m, &m->d_token, 16));
    LB_TRY(dalloc(m, &m->d_pos, 16));
    LB_TRY(dalloc(m, &m->d_next, 16));
    LB_TRY(dalloc(m, &m->cand_val, (size_t)lb_dense_ctas(c, m->vocab_s, H) * 4));
    LB_TRY(dalloc(m, &m->cand_idx, (size_t)lb_dense_ctas(c, m->vocab_s, H) * 4));
    LB_CU(c, lb_drv.MemHostAlloc((void**)&m->h_next, 64, 0));
    for (int l = 0; l < cfg->n_layers; l++) {
        layer_t* L = &m->L[l];
        L->is_fa = is_fa(cfg, l);
        if (L->is_fa) {
            size_t n = (size_t)cfg->max_ctx * m->HKV * 256 * 2;
            LB_TRY(dalloc(m, &L->k_cache, n));
            LB_TRY(dalloc(m, &L->v_cache, n));
        } else {
            LB_TRY(dalloc(m, &L->dn_state, (size_t)m->HV * 128 * 128 * 4));
            LB_TRY(dalloc(m, &L->conv_ring, (size_t)4 * m->C_s * 4));
        }
    }
    return lb_model_reset_state(m);
}

LB_API int lb_model_reset_state(lb_model* m) {
    if (!m) return LB_ERR_INVALID;
    lb_ctx* c = m->c;
    for (int l = 0; l < m->cfg.n_layers; l++) {
        layer_t* L = &m->L[l];
        if (L->is_fa) {
            size_t n = (size_t)m->cfg.max_ctx * m->HKV * 256 * 2;
            LB_CU(c, lb_drv.MemsetD8Async(L->k_cache, 0, n, c->stream));
            LB_CU(c, lb_drv.MemsetD8Async(L->v_cache, 0, n, c->stream));
        } else {
            LB_CU(c, lb_drv.MemsetD8Async(L->dn_state, 0, (size_t)m->HV * 128 * 128 * 4, c->stream));
            LB_CU(c, lb_drv.MemsetD8Async(L->conv_ring, 0, (size_t)4 * m->C_s * 4, c->stream));
        }
    }
    LB_CU(c, lb_drv.StreamSynchronize(c->stream));
    return LB_OK;
}

/* Checkpoint / rollback of the recurrent state: the reference's state_rollback kernel is an element-wise copy
 * state[i] = checkpoint[i] (inference/recur.ls:82-86, kernels/recurrence_rollback.sass).  Here both directions
 * are device-to-device copies of every DeltaNet layer's state matrix and convolution history on the context
 * stream (ordered with the decode steps around them).  The KV caches need no copy: a row is rewritten when
 * its position is decoded again, and rows past the current position are never read. */
static int model_snapshot(lb_model* m, int restore) {
    lb_ctx* c = m->c;
    const size_t sb = (size_t)m->HV * 128 * 128 * 4, cb = (size_t)4 * m->C_s * 4;
    for (int l = 0; l < m->cfg.n_layers; l++) {
        layer_t* L = &m->L[l];
        if (L->is_fa) continue;
        if (!L->snap_state) {
            if (restore) return lb_fail(c, LB_ERR_STATE, "lb_model_rollback: no checkpoint taken");
            LB_CU(c, lb_drv.MemAlloc(&L->snap_state, sb));
            LB_CU(c, lb_drv.MemAlloc(&L->snap_conv, cb));
        }
        if (restore) {
            LB_CU(c, lb_drv.MemcpyDtoDAsync(L->dn_state, L->snap_state, sb, c->stream));
            LB_CU(c, lb_drv.MemcpyDtoDAsync(L->conv_ring, L->snap_conv, cb, c->stream));
        } else {
            LB_CU(c, lb_drv.MemcpyDtoDAsync(L->snap_state, L->dn_state, sb, c->stream));
            LB_CU(c, lb_drv.MemcpyDtoDAsync(L->snap_conv, L->conv_ring, cb, c->stream));
        }
    }
    return LB_OK;
}
LB_API int lb_model_checkpoint(lb_model* m) { return m ? model_snapshot(m, 0) : LB_ERR_INVALID; }
LB_API int lb_model_rollback(lb_model* m) { return m ? model_snapshot(m, 1) : LB_ERR_INVALID; }

LB_API int lb_model_state_ptr(lb_model* m, int layer, int which, uint64_t* dptr, size_t* bytes) {
    if (!m || layer < 0 || layer >= m->cfg.n_layers || !dptr || !bytes || which < 0 || which > 1) return LB_ERR_INVALID;
    layer_t* L = &m->L[layer];
    if (L->is_fa) {
        *dptr = which ? L->v_cache : L->k_cache;
        *bytes = (size_t)m->cfg.max_ctx * m->HKV * 256 * 2;
    } else {
        *dptr = which ? L->conv_ring : L->dn_state;
        *bytes = which ? (size_t)4 * m->C_s * 4 : (size_t)m->HV * 128 * 128 * 4;
    }
    return LB_OK;
}
LB_API int lb_model_logits_ptr(lb_model* m, uint64_t* dptr) {
    if (!m || !dptr) return LB_ERR_INVALID;
    *dptr = m->logits;
    return LB_OK;
}
LB_API uint64_t lb_model_weight_bytes(const lb_model* m) { return m ? m->weight_bytes : 0; }
LB_API const lb_model_cfg* lb_model_config(const lb_model* m) { return m ? &m->cfg : NULL; }
LB_API int lb_model_step_kernels(const lb_model* m) { return m ? m->step_kernels : 0; }

/* ---- weight re-layout (host) --------------------------------------------------------
 * A "column map" lists, for every output column of the device matrix, the column of which
 * source matrix it comes from.  qweight / scales are gathered column by column; qzeros is
 * re-packed nibble by nibble (8 columns per word). */
typedef struct {
    const uint32_t* qw; const uint16_t* sc; const uint32_t* qz; int N;
    int synth;             /* the tensors are streams of the seeded generator (qw == sc == qz == NULL): elements are drawn on demand */
    uint64_t seed, stream; /* qweight = stream, scales = stream + 1, qzeros = stream + 2 */
} q4_src;
static inline uint32_t src_qw(const q4_src* s, size_t i) { return s->synth ? lb_rng_word(s->seed, s->stream, i) : s->qw[i]; }
static inline uint16_t src_sc(const q4_src* s, size_t i) { return s->synth ? lb_rng_scale_f16(s->seed, s->stream + 1, i) : s->sc[i]; }
static inline uint32_t src_qz(const q4_src* s, size_t i) { return s->synth ? lb_rng_word(s->seed, s->stream + 2, i) : s->qz[i]; }
/* seeded synthetic weights: tensor (layer, slot) is stream (layer + 1) * 100 + slot */
typedef struct { uint64_t seed, base; } synth_t;

/* gather one device matrix on the host: columns by map, packed rows of groups [k0,k1) */
static void gather_q4(const q4_src* src, const int* col_src, const int* col_idx, int N_out, int k0, int k1, uint32_t* qw,
                      uint16_t* sc, uint32_t* qz) {
    const int groups = k1 - k0, Kd = groups * 128;
    memset(qz, 0, (size_t)groups * (N_out / 8) * 4);
#pragma omp parallel for schedule(static)
    for (int kp = 0; kp < Kd / 8; kp++) {
        uint32_t* o = qw + (size_t)kp * N_out;
        for (int n = 0; n < N_out; n++) {
            const q4_src* s = &src[col_src[n]];
            o[n] = src_qw(s, (size_t)(k0 * 16 + kp) * s->N + col_idx[n]);
        }
    }
#pragma omp parallel for schedule(static)
    for (int g = 0; g < groups; g++) {
        for (int n = 0; n < N_out; n++) {
            const q4_src* s = &src[col_src[n]];
            int ci = col_idx[n];
            sc[(size_t)g * N_out + n] = src_sc(s, (size_t)(k0 + g) * s->N + ci);
            uint32_t z = (src_qz(s, (size_t)(k0 + g) * (s->N / 8) + (ci >> 3)) >> (4 * (ci & 7))) & 0xFu;
            qz[(size_t)g * (N_out / 8) + (n >> 3)] |= z << (4 * (n & 7));
        }
    }
}

static int build_q4(lb_model* m, q4_mat* dst, const q4_src* src, const int* col_src, const int* col_idx, int N_out, int k0,
                    int k1) {
    int groups = k1 - k0, Kd = groups * 128;
    size_t qb = (size_t)Kd / 8 * N_out * 4, sb = (size_t)groups * N_out * 2, zb = (size_t)groups * (N_out / 8) * 4;
    uint32_t* qw = (uint32_t*)malloc(qb);
    uint16_t* sc = (uint16_t*)malloc(sb);
    uint32_t* qz = (uint32_t*)malloc(zb);
    if (!qw || !sc || !qz) { free(qw); free(sc); free(qz); return lb_fail(m->c, LB_ERR_NOMEM, "model: host staging"); }
    gather_q4(src, col_src, col_idx, N_out, k0, k1, qw, sc, qz);
    dst->K = Kd; dst->N = N_out;
    int st = upload(m, &dst->qweight, qw, qb);
    if (st == LB_OK) st = upload(m, &dst->scales, sc, sb);
    if (st == LB_OK) st = upload(m, &dst->qzeros, qz, zb);
    free(qw); free(sc); free(qz);
    m->weight_bytes += qb + sb + zb;
    return st;
}

static q4_src slot_src(const void* const* slots, int base, int N, const synth_t* syn) {
    q4_src s;
    memset(&s, 0, sizeof s);
    s.N = N;
    if (syn) { s.synth = 1; s.seed = syn->seed; s.stream = syn->base + (uint64_t)base; }
    else { s.qw = (const uint32_t*)slots[base]; s.sc = (const uint16_t*)slots[base + 1]; s.qz = (const uint32_t*)slots[base + 2]; }
    return s;
}
static int slots_present(lb_model* m, const void* const* slots, const int* idx, int n, int layer) {
    for (int i = 0; i < n; i++)
        if (!slots[idx[i]]) return lb_fail(m->c, LB_ERR_INVALID, "model: layer %d weight slot %d is NULL", layer, idx[i]);
    return LB_OK;
}

/* copy rows [r0, r0+rows) of a row-major host matrix with `row_bytes` per row */
static int upload_rows(lb_model* m, CUdeviceptr* p, const void* src, size_t r0, size_t rows, size_t row_bytes) {
    return upload(m, p, (const unsigned char*)src + r0 * row_bytes, rows * row_bytes);
}

/* Which columns / packed-row groups of the reference's per-projection tensors make up device
 * matrix `which` (0 input projections fused, 1 output projection, 2 gate|up, 3 down) of shard
 * R of T.  Column-parallel matrices keep all of K and take the shard's heads / intermediate
 * columns; row-parallel ones keep all N and take the K groups of the shard's heads. */
typedef struct { q4_src src[3]; int* cs; int* ci; int N, k0, k1; } shard_plan;

static void plan_free(shard_plan* p) { free(p->cs); free(p->ci); p->cs = p->ci = NULL; }

static int plan_make(const lb_model_cfg* c, int R, int T, int fa, int which, const void* const* slots, const synth_t* syn, shard_plan* p) {
    memset(p, 0, sizeof *p);
    const int H = c->hidden, I = c->inter;
    const int HV = c->dn_v_heads / T, HK = c->dn_k_heads / T, HQ = c->fa_q_heads / T;
    const int HKV = c->fa_kv_heads >= T ? c->fa_kv_heads / T : 1;
    const int Is = I / T;
    int N = 0;
    if (which == 0 && !fa) {
        const int QKf = c->dn_k_heads * 128, Cf = (2 * c->dn_k_heads + c->dn_v_heads) * 128, Vf = c->dn_v_heads * 128;
        const int QK = HK * 128, V = HV * 128, C = 2 * QK + V;
        N = C + V;
        p->src[0] = slot_src(slots, WS_DN_QKV, Cf, syn); p->src[1] = slot_src(slots, WS_DN_Z, Vf, syn);
        p->cs = (int*)malloc(sizeof(int) * N); p->ci = (int*)malloc(sizeof(int) * N);
        if (!p->cs || !p->ci) return LB_ERR_NOMEM;
        for (int n = 0; n < N; n++) { /* device columns: q | k | v | z of this shard's heads */
            if (n < QK) { p->cs[n] = 0; p->ci[n] = R * QK + n; }
            else if (n < 2 * QK) { p->cs[n] = 0; p->ci[n] = QKf + R * QK + (n - QK); }
            else if (n < C) { p->cs[n] = 0; p->ci[n] = 2 * QKf + R * V + (n - 2 * QK); }
            else { p->cs[n] = 1; p->ci[n] = R * V + (n - C); }
        }
        p->k0 = 0; p->k1 = H / 128;
    } else if (which == 0) {
        const int NQf = 2 * c->fa_q_heads * 256, NKVf = c->fa_kv_heads * 256;
        const int NQ = 2 * HQ * 256, NKV = HKV * 256;
        const int kv0 = c->fa_kv_heads >= T ? R * HKV : (R * c->fa_kv_heads) / T; /* first KV head of this shard */
        N = NQ + 2 * NKV;
        p->src[0] = slot_src(slots, WS_FA_Q, NQf, syn); p->src[1] = slot_src(slots, WS_FA_K, NKVf, syn); p->src[2] = slot_src(slots, WS_FA_V, NKVf, syn);
        p->cs = (int*)malloc(sizeof(int) * N); p->ci = (int*)malloc(sizeof(int) * N);
        if (!p->cs || !p->ci) return LB_ERR_NOMEM;
        for (int n = 0; n < N; n++) { /* per query head 512 columns (query, gate), then the KV head(s) */
            if (n < NQ) { p->cs[n] = 0; p->ci[n] = R * NQ + n; }
            else if (n < NQ + NKV) { p->cs[n] = 1; p->ci[n] = kv0 * 256 + (n - NQ); }
            else { p->cs[n] = 2; p->ci[n] = kv0 * 256 + (n - NQ - NKV); }
        }
        p->k0 = 0; p->k1 = H / 128;
    } else if (which == 2) {
        N = 2 * Is;
        p->src[0] = slot_src(slots, WS_GATE, I, syn); p->src[1] = slot_src(slots, WS_UP, I, syn);
        p->cs = (int*)malloc(sizeof(int) * N); p->ci = (int*)malloc(sizeof(int) * N);
        if (!p->cs || !p->ci) return LB_ERR_NOMEM;
        for (int n = 0; n < N; n++) { int blk = n / 64; p->cs[n] = blk & 1; p->ci[n] = R * Is + (blk >> 1) * 64 + n % 64; }
        p->k0 = 0; p->k1 = H / 128;
    } else { /* row-parallel: out / o projection (which 1), down projection (which 3) */
        N = H;
        p->src[0] = slot_src(slots, which == 3 ? WS_DOWN : (fa ? WS_FA_O : WS_DN_OUT), H, syn);
        p->cs = (int*)calloc((size_t)N, sizeof(int)); p->ci = (int*)malloc(sizeof(int) * N);
        if (!p->cs || !p->ci) return LB_ERR_NOMEM;
        for (int n = 0; n < N; n++) p->ci[n] = n;
        if (which == 3) { p->k0 = R * Is / 128; p->k1 = (R + 1) * Is / 128; }
        else if (fa) { p->k0 = R * HQ * 2; p->k1 = (R + 1) * HQ * 2; }   /* two groups of 128 per 256-wide head */
        else { p->k0 = R * HV; p->k1 = (R + 1) * HV; }                    /* one group per value head */
    }
    p->N = N;
    return LB_OK;
}

/* Host-only view of the sharder (no GPU): sizes first (outputs NULL), then the data. */
LB_API int lb_model_shard_host(const lb_model_cfg* cfg, int tp_rank, int tp_size, int layer, int which,
                               const void* const* slots, uint32_t* qweight_out, uint16_t* scales_out, uint32_t* qzeros_out,
                               int* K_out, int* N_out) {
    if (!cfg || !slots || which < 0 || which > 3 || tp_size < 1 || tp_rank < 0 || tp_rank >= tp_size) return LB_ERR_INVALID;
    shard_plan p;
    int st = plan_make(cfg, tp_rank, tp_size, is_fa(cfg, layer), which, slots, NULL, &p);
    if (st == LB_OK) {
        if (K_out) *K_out = (p.k1 - p.k0) * 128;
        if (N_out) *N_out = p.N;
        if (qweight_out && scales_out && qzeros_out) gather_q4(p.src, p.cs, p.ci, p.N, p.k0, p.k1, qweight_out, scales_out, qzeros_out);
    }
    plan_free(&p);
    return st;
}

/* syn != NULL: the int4 tensors (slots 0-8 or 0-11, and 15-23) are not in `slots` but drawn from the generator */
static int load_layer(lb_model* m, int layer, const void* const* slots, const synth_t* syn) {
    if (!m || !slots || layer < 0 || layer >= m->cfg.n_layers) return LB_ERR_INVALID;
    const lb_model_cfg* c = &m->cfg;
    layer_t* L = &m->L[layer];
    if (L->loaded) return lb_fail(m->c, LB_ERR_STATE, "model: layer %d already loaded", layer);
    LB_CU(m->c, lb_drv.CtxSetCurrent(m->c->cu_ctx));
    const int H = c->hidden, R = m->tp_rank, T = m->tp_size;
    if (syn) {
        static const int need_dn[] = {9, 10, 11, 12, 13, 14, 24, 25}, need_fa[] = {12, 13, 24, 25};
        LB_TRY(slots_present(m, slots, L->is_fa ? need_fa : need_dn, L->is_fa ? 4 : 8, layer));
    } else if (!L->is_fa) {
        static const int need[] = {0, 1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11, 12, 13, 14, 15, 16, 17, 18, 19, 20, 21, 22, 23, 24, 25};
        LB_TRY(slots_present(m, slots, need, 26, layer));
    } else {
        static const int need[] = {0, 1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11, 12, 13, 15, 16, 17, 18, 19, 20, 21, 22, 23, 24, 25};
        LB_TRY(slots_present(m, slots, need, 25, layer));
    }
    q4_mat* mats[4] = {&L->w_in, &L->w_out, &L->w_gateup, &L->w_down};
    for (int which = 0; which < 4; which++) {
        shard_plan p;
        int st = plan_make(c, R, T, L->is_fa, which, slots, syn, &p);
        if (st == LB_OK) st = build_q4(m, mats[which], p.src, p.cs, p.ci, p.N, p.k0, p.k1);
        if (st == LB_OK && lb_gemv_chain_supports(m->c, mats[which]->K, mats[which]->N, which == 2) == LB_OK) {
            /* second copy in the chain kernel's layout: every SM's columns contiguous */
            q4_mat* w = mats[which];
            st = dalloc(m, &w->packed, lb_gemv_packed_bytes(w->K, w->N));
            if (st == LB_OK) st = lb_gemv_pack(m->c, w->qweight, w->scales, w->qzeros, w->K, w->N, which == 2, w->packed);
        }
        if (st == LB_OK && which == 0 && !L->is_fa) { /* conv taps of the shard's channels: the first C device columns */
            const int C = m->C_s, Cf = (2 * c->dn_k_heads + c->dn_v_heads) * 128;
            uint16_t* cw = (uint16_t*)malloc((size_t)4 * C * 2);
            if (!cw) st = LB_ERR_NOMEM;
            else {
                for (int t = 0; t < 4; t++)
                    for (int n = 0; n < C; n++) cw[(size_t)t * C + n] = ((const uint16_t*)slots[WS_DN_CONV1D])[(size_t)t * Cf + p.ci[n]];
                st = upload(m, &L->conv_w, cw, (size_t)4 * C * 2);
                free(cw);
            }
        }
        plan_free(&p);
        if (st != LB_OK) return st == LB_ERR_NOMEM ? lb_fail(m->c, st, "model: host staging") : st;
    }
    if (!L->is_fa) {
        LB_TRY(upload_rows(m, &L->proj_a, slots[WS_DN_PROJ_A], (size_t)R * m->HV, (size_t)m->HV, (size_t)H * 2));
        LB_TRY(upload_rows(m, &L->proj_b, slots[WS_DN_PROJ_B], (size_t)R * m->HV, (size_t)m->HV, (size_t)H * 2));
        LB_TRY(upload_rows(m, &L->a_log, slots[WS_DN_A_LOG], (size_t)R * m->HV, (size_t)m->HV, 4));
        LB_TRY(upload_rows(m, &L->dt_bias, slots[WS_DN_DT_BIAS], (size_t)R * m->HV, (size_t)m->HV, 2));
        LB_TRY(upload(m, &L->dn_norm, slots[WS_DN_NORM], 128 * 4));
        m->weight_bytes += (uint64_t)2 * m->HV * H * 2 + (uint64_t)4 * m->C_s * 2;
    } else {
        LB_TRY(upload(m, &L->q_norm, slots[WS_FA_Q_NORM], 256 * 2));
        LB_TRY(upload(m, &L->k_norm, slots[WS_FA_K_NORM], 256 * 2));
    }
    LB_TRY(upload(m, &L->input_norm, slots[WS_INPUT_NORM], (size_t)H * 2));
    LB_TRY(upload(m, &L->post_norm, slots[WS_POST_NORM], (size_t)H * 2));
    if (!L->is_fa) { /* the mixer's parameter block, for the persistent chain (read by the kernel from device memory) */
        lb_dn_layer_params dp;
        dn_fill_params(m, L, &dp);
        LB_TRY(upload(m, &L->dn_params, &dp, sizeof dp));
    }
    L->loaded = 1;
    return LB_OK;
}

LB_API int lb_model_load_layer(lb_model* m, int layer, const void* const* slots) { return load_layer(m, layer, slots, NULL); }

LB_API int lb_model_load_globals(lb_model* m, const void* const* g) {
    if (!m || !g || !g[0] || !g[1] || !g[2]) return LB_ERR_INVALID;
    if (m->globals_loaded) return lb_fail(m->c, LB_ERR_STATE, "model: globals already loaded");
    LB_CU(m->c, lb_drv.CtxSetCurrent(m->c->cu_ctx));
    size_t tb = (size_t)m->cfg.vocab * m->cfg.hidden * 2;
    LB_TRY(upload(m, &m->embed, g[WG_EMBED], tb));
    LB_TRY(upload_rows(m, &m->lm_head, g[WG_LM_HEAD], (size_t)m->tp_rank * m->vocab_s, (size_t)m->vocab_s, (size_t)m->cfg.hidden * 2));
    LB_TRY(upload(m, &m->final_norm, g[WG_FINAL_NORM], (size_t)m->cfg.hidden * 2));
    m->weight_bytes += tb / m->tp_size; /* the LM head shard is streamed every step; the embedding contributes one row */
    m->globals_loaded = 1;
    return LB_OK;
}

/* ---- seeded synthetic weights ------------------------------------------------------------ */
LB_API int lb_model_fill_synthetic(lb_model* m, uint64_t seed) {
    if (!m) return LB_ERR_INVALID;
    const lb_model_cfg* c = &m->cfg;
    const size_t H = c->hidden;
    for (int l = 0; l < c->n_layers; l++) {
        void* s[LB_WS_SLOTS];
        memset(s, 0, sizeof s);
        const uint64_t base = (uint64_t)(l + 1) * 100;
        const int fa = is_fa(c, l);
        int ok = 1;
        const synth_t syn = {seed, base}; /* the int4 tensors: only this shard's elements are drawn, inside the re-layout */
        uint16_t* in_norm = (uint16_t*)malloc(H * 2); uint16_t* post_norm = (uint16_t*)malloc(H * 2);
        ok &= in_norm && post_norm;
        if (ok) {
            lb_fill_normal_bf16(in_norm, H, seed, base + WS_INPUT_NORM, 0.f, 0.02f);
            lb_fill_normal_bf16(post_norm, H, seed, base + WS_POST_NORM, 0.f, 0.02f);
        }
        s[WS_INPUT_NORM] = in_norm; s[WS_POST_NORM] = post_norm;
        if (ok && !fa) {
            const size_t HV = c->dn_v_heads, C = (size_t)(2 * c->dn_k_heads + c->dn_v_heads) * 128;
            uint16_t* pa = (uint16_t*)malloc(HV * H * 2); uint16_t* pb = (uint16_t*)malloc(HV * H * 2);
            float* alog = (float*)malloc(HV * 4); uint16_t* dtb = (uint16_t*)malloc(HV * 2);
            uint16_t* cw = (uint16_t*)malloc(4 * C * 2); float* hn = (float*)malloc(128 * 4);
            ok &= pa && pb && alog && dtb && cw && hn;
            if (ok) {
                lb_fill_normal_bf16(pa, HV * H, seed, base + WS_DN_PROJ_A, 0.f, 0.02f);
                lb_fill_normal_bf16(pb, HV * H, seed, base + WS_DN_PROJ_B, 0.f, 0.02f);
                lb_fill_uniform_f32(alog, HV, seed, base + WS_DN_A_LOG, 0.f, 2.7f);
                lb_fill_normal_bf16(dtb, HV, seed, base + WS_DN_DT_BIAS, 0.f, 0.1f);
                lb_fill_normal_bf16(cw, 4 * C, seed, base + WS_DN_CONV1D, 0.f, 0.3f);
                lb_fill_normal_f32(hn, 128, seed, base + WS_DN_NORM, 1.f, 0.02f);
            }
            s[WS_DN_PROJ_A] = pa; s[WS_DN_PROJ_B] = pb; s[WS_DN_A_LOG] = alog; s[WS_DN_DT_BIAS] = dtb;
            s[WS_DN_CONV1D] = cw; s[WS_DN_NORM] = hn;
        } else if (ok) {
            uint16_t* qn = (uint16_t*)malloc(256 * 2); uint16_t* kn = (uint16_t*)malloc(256 * 2);
            ok &= qn && kn;
            if (ok) {
                lb_fill_normal_bf16(qn, 256, seed, base + WS_FA_Q_NORM, 1.f, 0.02f);
                lb_fill_normal_bf16(kn, 256, seed, base + WS_FA_K_NORM, 1.f, 0.02f);
            }
            s[WS_FA_Q_NORM] = qn; s[WS_FA_K_NORM] = kn;
        }
        int st = ok ? load_layer(m, l, (const void* const*)s, &syn) : lb_fail(m->c, LB_ERR_NOMEM, "model: host staging");
        for (int i = 0; i < LB_WS_SLOTS; i++) free(s[i]);
        if (st != LB_OK) return st;
    }
    {
        size_t n = (size_t)c->vocab * H;
        uint16_t* e = (uint16_t*)malloc(n * 2); uint16_t* h = (uint16_t*)malloc(n * 2); uint16_t* fn = (uint16_t*)malloc(H * 2);
        int st = LB_ERR_NOMEM;
        if (e && h && fn) {
            lb_fill_normal_bf16(e, n, seed, 1, 0.f, 0.02f);
            lb_fill_normal_bf16(h, n, seed, 2, 0.f, 0.02f);
            lb_fill_normal_bf16(fn, H, seed, 3, 0.f, 0.02f);
            const void* g[3] = {e, h, fn};
            st = lb_model_load_globals(m, g);
        }
        free(e); free(h); free(fn);
        if (st != LB_OK) return st;
    }
    return LB_OK;
}

/* ---- the step ------------------------------------------------------------------------------ */
/* parameters of the DeltaNet mixer of one layer (between the qkvz projection and the out projection) */
static void dn_fill_params(const lb_model* m, const layer_t* L, lb_dn_layer_params* p) {
    memset(p, 0, sizeof *p);
    p->qkvz = (const float*)m->in_out; p->xn = (const uint16_t*)m->xn;
    p->proj_a = (const uint16_t*)L->proj_a; p->proj_b = (const uint16_t*)L->proj_b;
    p->a_log = (const float*)L->a_log; p->dt_bias = (const uint16_t*)L->dt_bias;
    p->conv_w = (const uint16_t*)L->conv_w; p->conv_ring = (float*)L->conv_ring;
    p->state = (float*)L->dn_state; p->out = (float*)m->mix_out; p->pos = (const int*)m->d_pos;
    p->HV = m->HV; p->HK = m->HK; p->hidden = m->cfg.hidden;
}

/* launch what has been collected so far as one persistent kernel */
static int flush_chain(lb_model* m) {
    int n = m->n_pend;
    m->n_pend = 0;
    return n ? lb_chain_launch(m->c, m->pend, n) : LB_OK;
}

/* add an entry to the pending chain; what is pending goes out first when the new entry no longer fits beside it */
static int chain_push(lb_model* m, const lb_chain_op* op) {
    if (m->n_pend > 0) {
        int fits = m->n_pend < LB_CHAIN_MAX_OPS;
        if (fits) {
            m->pend[m->n_pend] = *op;
            fits = lb_chain_fits(m->c, m->pend, m->n_pend + 1) == LB_OK;
        }
        if (!fits) LB_TRY(flush_chain(m));
    }
    m->pend[m->n_pend++] = *op;
    return LB_OK;
}

static int q4_gemv(lb_model* m, const q4_mat* w, CUdeviceptr x, CUdeviceptr y, int x_mode, int y_mode, CUdeviceptr aux0,
                   CUdeviceptr aux1, CUdeviceptr x_out) {
    if (m->use_chain && w->packed) {
        lb_gemv_op o;
        memset(&o, 0, sizeof o);
        o.packed = w->packed;
        o.x = x; o.y = y; o.aux0 = aux0; o.aux1 = aux1; o.x_out = x_out;
        o.K = w->K; o.N = w->N; o.x_mode = x_mode; o.y_mode = y_mode; o.eps = m->cfg.eps;
        lb_chain_op k;
        LB_TRY(lb_chain_fill_gemv(m->c, &k, &o, m->n_pend));
        return chain_push(m, &k);
    }
    LB_TRY(flush_chain(m));
    return lb_gemv_int4_fused(m->c, w->qweight, w->scales, w->qzeros, x, y, w->K, w->N, x_mode, y_mode, aux0, aux1, x_out,
                              m->cfg.eps);
}

/* output of a row-parallel projection: straight into the residual stream on one GPU; on several,
 * this GPU's partial goes to its exchange buffer and tp_allreduce_add folds all partials into X */
static int row_parallel(lb_model* m, const q4_mat* w, CUdeviceptr x, int x_mode, CUdeviceptr aux0, CUdeviceptr aux1) {
    if (m->tp_size == 1) return q4_gemv(m, w, x, m->X, x_mode, LB_Y_F32_ACCUM, aux0, aux1, 0);
    if (!m->comm) return lb_fail(m->c, LB_ERR_STATE, "model: tensor-parallel shard without exchange buffers (lb_model_set_comm)");
    if (m->use_chain && w->packed && m->tp_params[0]) {
        /* the exchange happens inside the projection's epilogue (LB_Y_TP_ALLREDUCE): no entry or launch of its own */
        lb_gemv_op o;
        memset(&o, 0, sizeof o);
        o.packed = w->packed;
        o.x = x; o.y = m->X; o.aux0 = aux0; o.aux1 = aux1;
        o.K = w->K; o.N = w->N; o.x_mode = x_mode; o.y_mode = LB_Y_F32_ACCUM; o.eps = m->cfg.eps;
        lb_chain_op k;
        LB_TRY(lb_chain_fill_gemv(m->c, &k, &o, m->n_pend));
        k.y_mode = LB_Y_TP_ALLREDUCE;
        k.ext = (const void*)m->tp_params[0];
        return chain_push(m, &k);
    }
    const int slot = m->ar_count++ & 1;
    LB_TRY(q4_gemv(m, w, x, (CUdeviceptr)lb_comm_slot_ptr(m->comm, slot), x_mode, LB_Y_F32, aux0, aux1, 0));
    LB_TRY(flush_chain(m));
    lb_tp_params p;
    LB_TRY(lb_comm_fill(m->comm, &p, slot, m->cfg.hidden));
    p.x = (float*)m->X;
    void* params[] = {&p};
    return lb_launch(m->c, LBK_tp_allreduce_add, 1, 1, 1, 1024, 0, params, 1);
}

int lb_model_is_fa(const lb_model_cfg* c, int l) { return is_fa(c, l); }

int lb_model_launch_attention(lb_model* m, const layer_t* L, CUdeviceptr proj_row, CUdeviceptr out, CUdeviceptr pos_ptr, int pos, int splits_for) {
    lb_ctx* c = m->c;
    const lb_model_cfg* cfg = &m->cfg;
    lb_attn_params p;
    memset(&p, 0, sizeof p);
    const size_t nq = (size_t)2 * m->HQ * 256, nkv = (size_t)m->HKV * 256;
    p.q = (const void*)proj_row;                      /* per head: 256 query then 256 gate columns */
    p.gate = (const void*)(proj_row + 256 * 4);
    p.k_new = (const void*)(proj_row + nq * 4);
    p.v_new = (const void*)(proj_row + (nq + nkv) * 4);
    p.q_norm_w = (const uint16_t*)L->q_norm; p.k_norm_w = (const uint16_t*)L->k_norm;
    p.k_cache = (uint16_t*)L->k_cache; p.v_cache = (uint16_t*)L->v_cache;
    p.out = (float*)out; p.scratch = (float*)c->attn_scratch;
    p.counters = (uint32_t*)(c->gemv_counters + 2048 * 4);
    p.pos_ptr = (const int*)pos_ptr; p.pos = pos;
    p.HQ = m->HQ; p.HKV = m->HKV;
    p.splits = lb_attn_mma_splits(c, splits_for, m->HKV);
    p.status = (uint32_t*)c->dev_status;
    p.coop = m->HKV * p.splits <= c->sm_count;
    p.max_ctx = cfg->max_ctx;
    p.in_dtype = 1; p.gate_stride = 512; p.q_stride = 512;
    p.rot_dims = cfg->rot_dims; p.rope_theta = cfg->rope_theta; p.eps = cfg->eps;
    for (int i = 0; i < cfg->rot_dims / 2; i++)
        p.rope_freq[i] = exp2(-log2((double)cfg->rope_theta) * (double)i / (double)(cfg->rot_dims / 2));
    void* params[] = {&p};
    return lb_launch(c, LBK_attn_decode_mma, (unsigned)m->HKV, (unsigned)p.splits, 1, 256, lb_attn_mma_smem(m->HQ / m->HKV), params, 1);
}

/* the kernel that turns the LM head's output into the next token (and advances the position on the device) */
int lb_model_launch_sampler(lb_model* m) {
    lb_ctx* c = m->c;
    const int H = m->cfg.hidden;
    if (m->tp_size == 1 && m->top_k > 0) { /* temperature / top-k sampling over the full logits; the draw is a function of (seed, position) */
        uint64_t zero = 0;
        int n = m->vocab_s;
        void* params[] = {&m->logits, &n, &m->d_next, &m->d_token, &m->d_pos, &m->temperature, &m->top_k, &m->sample_seed, &zero, &zero, &zero};
        LB_TRY(lb_launch(c, LBK_topk_sample_f32, 1, 1, 1, 1024, 0, params, 1));
    } else if (m->tp_size == 1) {
        int n = lb_dense_ctas(c, m->vocab_s, H); /* one (value, row) candidate per LM-head CTA */
        void* params[] = {&m->cand_val, &n, &m->d_next, &m->d_token, &m->d_pos, &m->cand_idx};
        LB_TRY(lb_launch(c, LBK_argmax_f32, 1, 1, 1, 1024, 0, params, 1));
    } else {
        lb_tp_argmax_params q;
        memset(&q, 0, sizeof q);
        LB_TRY(lb_comm_fill(m->comm, &q.tp, 2, 2));
        q.cand_val = (const float*)m->cand_val; q.cand_idx = (const int32_t*)m->cand_idx;
        q.n_cand = lb_dense_ctas(c, m->vocab_s, H); q.vocab_offset = m->tp_rank * m->vocab_s;
        q.out_idx = (int32_t*)m->d_next; q.next_token = (int32_t*)m->d_token; q.pos = (int32_t*)m->d_pos;
        void* params[] = {&q};
        LB_TRY(lb_launch(c, LBK_tp_argmax_exchange, 1, 1, 1, 1024, 0, params, 1));
    }
    return LB_OK;
}

static int issue_step(lb_model* m) {
    lb_ctx* c = m->c;
    const lb_model_cfg* cfg = &m->cfg;
    const int H = cfg->hidden;
    uint64_t launches0 = c->launches;
    m->ar_count = 0;
    m->n_pend = 0;
    {
        void* params[] = {&m->embed, &m->d_token, &m->X, (void*)&H};
        LB_TRY(lb_launch(c, LBK_embed_bf16, (unsigned)((H + 1023) / 1024), 1, 1, 256, 0, params, 1));
    }
    for (int l = 0; l < cfg->n_layers; l++) {
        layer_t* L = &m->L[l];
        if (!L->loaded) return lb_fail(c, LB_ERR_STATE, "model: layer %d has no weights", l);
        if (!L->is_fa) {
            const int C = m->C_s;
            LB_TRY(q4_gemv(m, &L->w_in, m->X, m->in_out, LB_X_F32_RMSNORM, LB_Y_F32, L->input_norm, 0, m->xn));
            lb_dn_layer_params p;
            dn_fill_params(m, L, &p);
            if (m->use_chain && L->dn_params && L->w_in.packed) { /* the mixer joins the persistent chain */
                lb_chain_op k;
                memset(&k, 0, sizeof k);
                k.type = LB_CHAIN_OP_DELTANET;
                k.ext = (const void*)L->dn_params;
                LB_TRY(chain_push(m, &k));
            } else {
                void* params[] = {&p};
                LB_TRY(flush_chain(m));
                LB_TRY(lb_launch(c, LBK_deltanet_layer_fused, (unsigned)m->HV, 4, 1, 128, 0, params, 1));
            }
            LB_TRY(row_parallel(m, &L->w_out, m->mix_out, LB_X_F32_HEADNORM_SILU, L->dn_norm, m->in_out + (size_t)C * 4));
        } else {
            LB_TRY(q4_gemv(m, &L->w_in, m->X, m->in_out, LB_X_F32_RMSNORM, LB_Y_F32, L->input_norm, 0, 0));
            LB_TRY(flush_chain(m));
            LB_TRY(lb_model_launch_attention(m, L, m->in_out, m->mix_out, m->d_pos, 0, cfg->max_ctx));
            LB_TRY(row_parallel(m, &L->w_out, m->mix_out, LB_X_F32, 0, 0));
        }
        LB_TRY(q4_gemv(m, &L->w_gateup, m->X, m->mlp_m, LB_X_F32_RMSNORM, LB_Y_SWIGLU_F16, L->post_norm, 0, 0));
        LB_TRY(row_parallel(m, &L->w_down, m->mlp_m, LB_X_F16, 0, 0));
    }
    if (!m->globals_loaded) return lb_fail(c, LB_ERR_STATE, "model: globals have no weights");
    LB_TRY(flush_chain(m));
    LB_TRY(lb_dense_launch(c, m->lm_head, m->X, m->logits, m->vocab_s, H, LB_X_F32_RMSNORM, m->final_norm, cfg->eps,
                           m->cand_val, m->cand_idx));
    LB_TRY(lb_model_launch_sampler(m));
    m->step_kernels = (int)(c->launches - launches0);
    return LB_OK;
}

/* top_k == 0 (default): greedy.  Otherwise the step samples among the top_k largest logits at this temperature; the
 * uniform draw of a step is element (position) of a stream of the seeded generator, so a run can be repeated.  Takes
 * effect at the next lb_model_decode / lb_model_capture.  Single GPU only. */
LB_API int lb_model_set_sampling(lb_model* m, float temperature, int top_k, uint64_t seed) {
    if (!m) return LB_ERR_INVALID;
    if (top_k < 0 || top_k > 64 || (top_k > 0 && !(temperature > 0.f))) return lb_fail(m->c, LB_ERR_INVALID, "model: sampling needs 0 <= top_k <= 64 and temperature > 0");
    if (top_k > 0 && m->tp_size != 1) return lb_fail(m->c, LB_ERR_STATE, "model: sampling other than greedy is single-GPU only");
    m->temperature = temperature; m->top_k = top_k; m->sample_seed = seed;
    if (m->graph) { lb_graph_destroy(m->c, m->graph); m->graph = NULL; } /* a captured step samples the old way */
    return LB_OK;
}

LB_API int lb_model_set_chain(lb_model* m, int on) {
    if (!m) return LB_ERR_INVALID;
    m->use_chain = on ? 1 : 0;
    return LB_OK;
}

LB_API int lb_model_set_comm(lb_model* m, lb_comm* comm) {
    if (!m || !comm) return LB_ERR_INVALID;
    if (lb_comm_rank(comm) != m->tp_rank || lb_comm_size(comm) != m->tp_size)
        return lb_fail(m->c, LB_ERR_INVALID, "model: exchange buffers are for rank %d/%d, the model is shard %d/%d",
                       lb_comm_rank(comm), lb_comm_size(comm), m->tp_rank, m->tp_size);
    m->comm = comm;
    for (int slot = 0; slot < 2; slot++) { /* the exchange parameters of both slots, for all-reduce entries of the chain */
        lb_tp_params p;
        LB_TRY(lb_comm_fill(comm, &p, slot, m->cfg.hidden));
        p.x = (float*)m->X;
        if (m->tp_params[slot]) { lb_drv.MemFree(m->tp_params[slot]); m->tp_params[slot] = 0; }
        LB_TRY(upload(m, &m->tp_params[slot], &p, sizeof p));
    }
    return LB_OK;
}

LB_API int lb_model_set_input(lb_model* m, int token, int pos) {
    if (!m) return LB_ERR_INVALID;
    if (token < 0 || token >= m->cfg.vocab || pos < 0 || pos >= m->cfg.max_ctx)
        return lb_fail(m->c, LB_ERR_INVALID, "model: token %d / position %d out of range", token, pos);
    /* by value, in stream order: back-to-back calls cannot overwrite each other's staging */
    LB_CU(m->c, lb_drv.MemsetD32Async(m->d_token, (unsigned)token, 1, m->c->stream));
    LB_CU(m->c, lb_drv.MemsetD32Async(m->d_pos, (unsigned)pos, 1, m->c->stream));
    m->host_pos = pos;
    return LB_OK;
}

LB_API int lb_model_read_next(lb_model* m, int* next_out) {
    if (!m || !next_out) return LB_ERR_INVALID;
    LB_CU(m->c, lb_drv.MemcpyDtoHAsync(&m->h_next[0], m->d_next, 4, m->c->stream));
    LB_CU(m->c, lb_drv.StreamSynchronize(m->c->stream));
    *next_out = m->h_next[0];
    uint32_t st = 0;
    return lb_device_status(m->c, &st);
}

LB_API int lb_model_decode(lb_model* m, int token, int pos, int* next_out) {
    if (!m || !next_out) return LB_ERR_INVALID;
    LB_CU(m->c, lb_drv.CtxSetCurrent(m->c->cu_ctx));
    LB_TRY(lb_model_set_input(m, token, pos));
    LB_TRY(issue_step(m));
    m->host_pos = pos + 1;
    return lb_model_read_next(m, next_out);
}

LB_API int lb_model_capture(lb_model* m) {
    if (!m) return LB_ERR_INVALID;
    if (m->graph) { lb_graph_destroy(m->c, m->graph); m->graph = NULL; }
    LB_CU(m->c, lb_drv.CtxSetCurrent(m->c->cu_ctx));
    LB_TRY(lb_graph_begin_capture(m->c));
    int st = issue_step(m);
    lb_graph* g = NULL;
    int st2 = lb_graph_end_capture(m->c, &g);
    if (st != LB_OK) { if (g) lb_graph_destroy(m->c, g); return st; }
    if (st2 != LB_OK) return st2;
    m->graph = g;
    m->step_kernels = lb_graph_kernel_count(g);
    return LB_OK;
}

LB_API int lb_model_replay(lb_model* m, int n_steps) {
    if (!m || n_steps < 0) return LB_ERR_INVALID;
    if (!m->graph) return lb_fail(m->c, LB_ERR_STATE, "model: replay before capture");
    /* every step appends one KV row at its position and advances the position on the device: refuse what would run past
     * the caches before anything is launched */
    if (m->host_pos + n_steps > m->cfg.max_ctx)
        return lb_fail(m->c, LB_ERR_INVALID, "model: %d steps from position %d run past the context of %d rows", n_steps, m->host_pos,
                       m->cfg.max_ctx);
    for (int i = 0; i < n_steps; i++) {
        LB_TRY(lb_graph_launch(m->c, m->graph));
        m->host_pos++;
    }
    return LB_OK;
}

/* The launcher's decode loop (src/launcher.s:552-652 generation loop, :931-1087 sample and print): run the prompt, then
 * decode until `eos` (248044 for the reference model, models/families/qwen/qwen3.5/27b/config.json:12; negative = none) or
 * max_new tokens.  out receives the generated tokens (the end-of-sequence token included when it was produced). */
LB_API int lb_model_generate(lb_model* m, const int* prompt, int n_prompt, int max_new, int eos, int* out, int* n_out) {
    if (!m || !prompt || n_prompt < 1 || max_new < 0 || !out || !n_out) return LB_ERR_INVALID;
    *n_out = 0;
    if (max_new == 0) return LB_OK;
    int tok = 0;
    LB_TRY(lb_model_prefill(m, prompt, n_prompt, 0, &tok));
    out[(*n_out)++] = tok;
    if (!m->graph) LB_TRY(lb_model_capture(m));
    while (*n_out < max_new && tok != eos) {
        if (m->host_pos >= m->cfg.max_ctx) break; /* the context is full */
        LB_TRY(lb_model_replay(m, 1)); /* token and position are already on the device */
        LB_TRY(lb_model_read_next(m, &tok));
        out[(*n_out)++] = tok;
    }
    return LB_OK;
}

LB_API void lb_model_destroy(lb_model* m) {
    if (!m) return;
    lb_ctx* c = m->c;
    if (lb_drv.loaded && c && c->cu_ctx) {
        lb_drv.CtxSetCurrent(c->cu_ctx);
        lb_drv.StreamSynchronize(c->stream);
        if (m->graph) lb_graph_destroy(c, m->graph);
        CUdeviceptr g[] = {m->embed, m->lm_head, m->final_norm, m->X, m->xn, m->in_out, m->mix_out, m->mlp_m, m->logits,
                           m->d_token, m->d_pos, m->d_next, m->cand_val, m->cand_idx, m->tp_params[0], m->tp_params[1]};
        for (size_t i = 0; i < sizeof g / sizeof g[0]; i++) if (g[i]) lb_drv.MemFree(g[i]);
        for (int l = 0; m->L && l < m->cfg.n_layers; l++) {
            layer_t* L = &m->L[l];
            q4_mat* q[] = {&L->w_in, &L->w_out, &L->w_gateup, &L->w_down};
            for (int i = 0; i < 4; i++) {
                if (q[i]->qweight) lb_drv.MemFree(q[i]->qweight);
                if (q[i]->scales) lb_drv.MemFree(q[i]->scales);
                if (q[i]->qzeros) lb_drv.MemFree(q[i]->qzeros);
                if (q[i]->packed) lb_drv.MemFree(q[i]->packed);
            }
            CUdeviceptr p[] = {L->input_norm, L->post_norm, L->proj_a, L->proj_b, L->a_log, L->dt_bias, L->conv_w, L->dn_norm,
                               L->dn_state, L->conv_ring, L->q_norm, L->k_norm, L->k_cache, L->v_cache, L->dn_params,
                               L->snap_state, L->snap_conv};
            for (size_t i = 0; i < sizeof p / sizeof p[0]; i++) if (p[i]) lb_drv.MemFree(p[i]);
        }
        lb_prefill_ws_free(m);
        if (m->h_next) lb_drv.MemFreeHost(m->h_next);
    }
    free(m->L);
    free(m);
}
