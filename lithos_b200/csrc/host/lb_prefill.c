/* The prompt pass: lb_model_prefill runs n prompt tokens through the model in chunks of up to 256 and leaves the state a
 * token-by-token decode of the same tokens leaves (DeltaNet states, convolution rings, KV rows), then samples the token
 * that follows the prompt.
 *
 * The reference's prompt path is its dequantising tensor-core GEMM (kernels/projection_gemm.sass:390-631) in the layer
 * order of compiler/megakernel-link.ls:281-525.  Here every projection of a chunk is one lb_gemm_int4 call (the weights
 * are read once per chunk: tcgen05 for 33..256 tokens), the DeltaNet recurrence walks the chunk's tokens inside one
 * launch with the state held on chip (lb_deltanet_step, n_steps = chunk), and attention is two launches per chunk: the
 * per-token part (norm, RoPE, KV append) with the decode kernel's own routine, then one causal tensor-core kernel over
 * all the chunk's tokens (pf_attn_prepare, pf_attn_chunk).  Single GPU only.
 *
 * PF_STREAMS chunks are in flight at a time, each on its own stream with its own buffer set: chunk c+1 follows chunk c one layer behind
 * (layer l of chunk c+1 waits for the event recorded after layer l of chunk c: the DeltaNet state, the convolution ring and
 * the cache rows of a layer pass from chunk to chunk in order).  About half of a chunk-layer's time is kernels that
 * cannot fill the GPU (the recurrence: 192 small CTAs walking 256 dependent steps; chunk attention; the element-wise
 * kernels): they now run beside the other chunk's projections instead of alone.
 */
#include "lb_model_priv.h"
#include <math.h>

extern int lb_dense_launch(lb_ctx* c, uint64_t w, uint64_t x, uint64_t y, int N, int K, int x_mode, uint64_t norm_w, float eps,
                           uint64_t part_val, uint64_t part_idx);
extern int lb_dense_ctas(lb_ctx* c, int N, int K);

#define PF_CHUNK 256
#define PF_STREAMS 4 /* chunks in flight */

typedef struct { /* the activations of one chunk */
    CUdeviceptr X, xn16, proj, q, k, v, g, beta, mix, mix16, y, gu, act16;
} pf_set;
#define PF_SET_PTRS (sizeof(pf_set) / sizeof(CUdeviceptr))

struct lb_prefill_ws {
    pf_set set[PF_STREAMS]; /* one per stream */
    pf_set* cur;            /* the set of the chunk being enqueued */
    CUdeviceptr tokens;     /* the whole prompt's token ids [max_ctx] */
    CUstream stream[PF_STREAMS];
    CUevent* layer_done[PF_STREAMS]; /* [n_layers] per stream: recorded after a chunk's layer l */
    CUevent fork, join[PF_STREAMS];
};

void lb_prefill_ws_free(lb_model* m);

static int ws_fill(lb_model* m) {
    lb_prefill_ws* ws = (lb_prefill_ws*)calloc(1, sizeof *ws);
    if (!ws) return LB_ERR_NOMEM;
    m->ws = ws; /* ws_alloc releases whatever a failure below leaves behind */
    lb_ctx* ctx = m->c;
    const lb_model_cfg* c = &m->cfg;
    const size_t T = PF_CHUNK, H = (size_t)c->hidden, I = (size_t)m->inter_s;
    size_t n_in = (size_t)m->C_s + (size_t)m->HV * 128, n_fa = (size_t)(2 * m->HQ + 2 * m->HKV) * 256;
    if (n_fa > n_in) n_in = n_fa;
    size_t n_mix = (size_t)m->HV * 128 > (size_t)m->HQ * 256 ? (size_t)m->HV * 128 : (size_t)m->HQ * 256;
    uint64_t d = 0;
    LB_TRY(lb_malloc(ctx, (size_t)c->max_ctx * 4, &d));
    ws->tokens = (CUdeviceptr)d;
    for (int s = 0; s < PF_STREAMS; s++) {
        pf_set* w = &ws->set[s];
        struct { CUdeviceptr* p; size_t bytes; } a[] = {
            {&w->X, T * H * 4}, {&w->xn16, T * H * 2}, {&w->proj, T * n_in * 4},
            {&w->q, T * (size_t)m->HK * 128 * 4}, {&w->k, T * (size_t)m->HK * 128 * 4}, {&w->v, T * (size_t)m->HV * 128 * 4},
            {&w->g, T * (size_t)m->HV * 4}, {&w->beta, T * (size_t)m->HV * 4}, {&w->mix, T * n_mix * 4}, {&w->mix16, T * n_mix * 2},
            {&w->y, T * H * 4}, {&w->gu, T * 2 * I * 4}, {&w->act16, T * I * 2}};
        for (size_t i = 0; i < sizeof a / sizeof a[0]; i++) {
            LB_TRY(lb_malloc(ctx, a[i].bytes, &d));
            *a[i].p = (CUdeviceptr)d;
        }
        LB_CU(ctx, lb_drv.StreamCreate(&ws->stream[s], CU_STREAM_NON_BLOCKING));
        ws->layer_done[s] = (CUevent*)calloc((size_t)c->n_layers, sizeof(CUevent));
        if (!ws->layer_done[s]) return LB_ERR_NOMEM;
        for (int l = 0; l < c->n_layers; l++) LB_CU(ctx, lb_drv.EventCreate(&ws->layer_done[s][l], CU_EVENT_DISABLE_TIMING));
        LB_CU(ctx, lb_drv.EventCreate(&ws->join[s], CU_EVENT_DISABLE_TIMING));
    }
    LB_CU(ctx, lb_drv.EventCreate(&ws->fork, CU_EVENT_DISABLE_TIMING));
    return LB_OK;
}

static int ws_alloc(lb_model* m) {
    if (m->ws) return LB_OK;
    const int st = ws_fill(m);
    if (st != LB_OK) lb_prefill_ws_free(m); /* never leave half a workspace behind for the next call */
    return st;
}

void lb_prefill_ws_free(lb_model* m) {
    lb_prefill_ws* ws = m->ws;
    if (!ws) return;
    for (int s = 0; s < PF_STREAMS; s++) {
        if (ws->stream[s]) lb_drv.StreamSynchronize(ws->stream[s]);
        CUdeviceptr* p = (CUdeviceptr*)&ws->set[s];
        for (size_t i = 0; i < PF_SET_PTRS; i++)
            if (p[i]) lb_drv.MemFree(p[i]);
        if (ws->layer_done[s]) {
            for (int l = 0; l < m->cfg.n_layers; l++)
                if (ws->layer_done[s][l]) lb_drv.EventDestroy(ws->layer_done[s][l]);
            free(ws->layer_done[s]);
        }
        if (ws->join[s]) lb_drv.EventDestroy(ws->join[s]);
        if (ws->stream[s]) lb_drv.StreamDestroy(ws->stream[s]);
    }
    if (ws->fork) lb_drv.EventDestroy(ws->fork);
    if (ws->tokens) lb_drv.MemFree(ws->tokens);
    free(ws);
    m->ws = NULL;
}

static unsigned blocks_for(long long n) {
    long long b = (n + 255) / 256;
    return (unsigned)(b > 4096 ? 4096 : b < 1 ? 1 : b);
}

static int gemm(lb_model* m, const q4_mat* w, CUdeviceptr x16, CUdeviceptr y32, int T) {
    return lb_gemm_int4(m->c, w->qweight, w->scales, w->qzeros, x16, y32, w->K, w->N, T, LB_GEMV_Y_F32);
}

static int add_into_x(lb_model* m, int T) {
    pf_set* w = m->ws->cur;
    int n4 = T * m->cfg.hidden / 4;
    void* params[] = {&w->X, &w->y, &n4};
    return lb_launch(m->c, LBK_pf_add, blocks_for(n4), 1, 1, 256, 0, params, 1);
}

/* xn16 = fp16(rmsnorm(X)); with add_y the projection result in y is added into X first (the residual add in the same pass) */
static int norm_f16(lb_model* m, CUdeviceptr norm_w, int T, int add_y) {
    pf_set* w = m->ws->cur;
    int D = m->cfg.hidden;
    float eps = m->cfg.eps;
    CUdeviceptr add = add_y ? w->y : 0;
    void* params[] = {&w->X, &add, &norm_w, &w->xn16, &D, &eps};
    return lb_launch(m->c, LBK_pf_rmsnorm_f16, (unsigned)T, 1, 1, 256, 0, params, 1);
}

static int chunk_layer(lb_model* m, int l, int pos0, int T) {
    lb_ctx* c = m->c;
    pf_set* w = m->ws->cur;
    const lb_model_cfg* cfg = &m->cfg;
    layer_t* L = &m->L[l];
    const int H = cfg->hidden;
    if (!L->loaded) return lb_fail(c, LB_ERR_STATE, "model: layer %d has no weights", l);
    LB_TRY(norm_f16(m, L->input_norm, T, 0));
    LB_TRY(gemm(m, &L->w_in, w->xn16, w->proj, T));
    int ld = L->w_in.N;
    if (!L->is_fa) {
        const int C = m->C_s, HK = m->HK, HV = m->HV;
        {
            void* params[] = {&w->proj, &ld, &L->conv_w, &L->conv_ring, &w->q, &w->k, &w->v, (void*)&HK, (void*)&HV, &pos0, &T};
            LB_TRY(lb_launch(c, LBK_pf_dn_frontend, (unsigned)T, (unsigned)(2 * HK + HV), 1, 128, 0, params, 1));
        }
        {
            int Cq = 2 * HK * 128 + HV * 128;
            void* params[] = {&w->proj, &ld, &L->conv_ring, &Cq, &pos0, &T};
            LB_TRY(lb_launch(c, LBK_pf_dn_ring, (unsigned)((Cq + 255) / 256), 1, 1, 256, 0, params, 1));
        }
        {
            void* params[] = {&w->xn16, &L->proj_a, &L->proj_b, &L->a_log, &L->dt_bias, &w->g, &w->beta, (void*)&HV, (void*)&H, &T};
            LB_TRY(lb_launch(c, LBK_pf_ab_gate, (unsigned)((T + 7) / 8), (unsigned)HV, 1, 128, 0, params, 1));
        }
        LB_TRY(lb_deltanet_step(c, L->dn_state, w->q, w->k, w->v, 0, w->g, w->beta, w->mix, HV, HK, T, 1));
        {
            float eps = cfg->eps;
            int z_off = C;
            void* params[] = {&w->mix, &w->proj, &ld, &z_off, &L->dn_norm, &w->mix16, (void*)&HV, &eps};
            LB_TRY(lb_launch(c, LBK_pf_headnorm_gate_f16, (unsigned)T, (unsigned)((HV + 3) / 4), 1, 128, 0, params, 1));
        }
    } else {
        /* per token: norm, RoPE, the chunk's KV rows into the cache, queries as two bf16 terms (in the fp32 mixer buffer);
         * then every token of the chunk at once, token s over the cache rows [0, pos0 + s] */
        lb_pf_attn_params p;
        memset(&p, 0, sizeof p);
        p.proj = (const float*)w->proj;
        p.q_norm_w = (const uint16_t*)L->q_norm; p.k_norm_w = (const uint16_t*)L->k_norm;
        p.k_cache = (uint16_t*)L->k_cache; p.v_cache = (uint16_t*)L->v_cache;
        p.qh = (uint16_t*)w->mix; p.ql = (uint16_t*)(w->mix + (size_t)PF_CHUNK * m->HQ * 256 * 2);
        p.out = (uint16_t*)w->mix16;
        p.ld = ld; p.HQ = m->HQ; p.HKV = m->HKV; p.pos0 = pos0; p.T = T; p.rot_dims = cfg->rot_dims; p.eps = cfg->eps;
        for (int i = 0; i < cfg->rot_dims / 2; i++)
            p.rope_freq[i] = exp2(-log2((double)cfg->rope_theta) * (double)i / (double)(cfg->rot_dims / 2));
        void* params[] = {&p};
        LB_TRY(lb_launch(c, LBK_pf_attn_prepare, (unsigned)T, 1, 1, 256, 0, params, 1));
        const int rows = T * (m->HQ / m->HKV);
        LB_TRY(lb_launch(c, LBK_pf_attn_chunk, (unsigned)((rows + LB_PF_ATTN_ROWS - 1) / LB_PF_ATTN_ROWS), (unsigned)m->HKV, 1,
                         LB_PF_ATTN_THREADS, LB_PF_ATTN_SMEM, params, 1));
    }
    LB_TRY(gemm(m, &L->w_out, w->mix16, w->y, T));
    /* MLP */
    LB_TRY(norm_f16(m, L->post_norm, T, 1));
    LB_TRY(gemm(m, &L->w_gateup, w->xn16, w->gu, T));
    {
        int I = m->inter_s;
        int total4 = T * (I / 4);
        void* params[] = {&w->gu, &w->act16, &I, &total4};
        LB_TRY(lb_launch(c, LBK_pf_swiglu_f16, blocks_for(total4), 1, 1, 256, 0, params, 1));
    }
    LB_TRY(gemm(m, &L->w_down, w->act16, w->y, T));
    return add_into_x(m, T);
}

LB_API int lb_model_prefill(lb_model* m, const int* tokens, int n, int pos0, int* next_out) {
    if (!m || !tokens || n < 1 || pos0 < 0) return LB_ERR_INVALID;
    lb_ctx* c = m->c;
    const lb_model_cfg* cfg = &m->cfg;
    if (m->tp_size != 1) return lb_fail(c, LB_ERR_STATE, "lb_model_prefill: single GPU only (this model is shard %d of %d)", m->tp_rank, m->tp_size);
    if (pos0 + n > cfg->max_ctx) return lb_fail(c, LB_ERR_INVALID, "lb_model_prefill: %d tokens from position %d run past the context of %d rows", n, pos0, cfg->max_ctx);
    for (int i = 0; i < n; i++)
        if (tokens[i] < 0 || tokens[i] >= cfg->vocab) return lb_fail(c, LB_ERR_INVALID, "lb_model_prefill: token %d at %d out of range", tokens[i], i);
    if (!m->globals_loaded) return lb_fail(c, LB_ERR_STATE, "model: globals have no weights");
    LB_CU(c, lb_drv.CtxSetCurrent(c->cu_ctx));
    LB_TRY(ws_alloc(m));
    lb_prefill_ws* ws = m->ws;
    const int H = cfg->hidden;
    CUstream main_stream = c->stream;
    LB_CU(c, lb_drv.MemcpyHtoDAsync(ws->tokens, tokens, (size_t)n * 4, main_stream));
    LB_CU(c, lb_drv.StreamSynchronize(main_stream)); /* the caller's token array may be pageable */
    /* the chunk streams start behind what the caller's stream holds so far (an earlier decode step, the token copy) */
    LB_CU(c, lb_drv.EventRecord(ws->fork, main_stream));
    for (int s = 0; s < PF_STREAMS; s++) LB_CU(c, lb_drv.StreamWaitEvent(ws->stream[s], ws->fork, 0));
    int st = LB_OK, chunk = 0;
    for (int c0 = 0; c0 < n && st == LB_OK; c0 += PF_CHUNK, chunk++) {
        const int T = n - c0 < PF_CHUNK ? n - c0 : PF_CHUNK, s = chunk % PF_STREAMS, prev = (chunk + PF_STREAMS - 1) % PF_STREAMS;
        ws->cur = &ws->set[s];
        c->stream = ws->stream[s]; /* every launch below goes to this chunk's stream */
        CUdeviceptr toks = ws->tokens + (size_t)c0 * 4;
        void* params[] = {&m->embed, &toks, &ws->cur->X, (void*)&H};
        st = lb_launch(c, LBK_pf_embed, (unsigned)T, 1, 1, 256, 0, params, 1);
        for (int l = 0; l < cfg->n_layers && st == LB_OK; l++) {
            /* layer l's state, ring and cache rows come from the previous chunk's layer l (on the stream before this one) */
            if (chunk > 0 && lb_drv.StreamWaitEvent(c->stream, ws->layer_done[prev][l], 0) != CUDA_SUCCESS) st = LB_ERR_CUDA;
            if (st == LB_OK) st = chunk_layer(m, l, pos0 + c0, T);
            if (st == LB_OK && lb_drv.EventRecord(ws->layer_done[s][l], c->stream) != CUDA_SUCCESS) st = LB_ERR_CUDA;
        }
        if (st == LB_OK && c0 + T == n) { /* the last prompt token's hidden state -> final norm, LM head, greedy sample */
            if (lb_drv.MemcpyDtoDAsync(m->X, ws->cur->X + (size_t)(T - 1) * H * 4, (size_t)H * 4, c->stream) != CUDA_SUCCESS) st = LB_ERR_CUDA;
        }
    }
    c->stream = main_stream;
    /* the caller's stream continues behind all chunk streams (also after a failed launch: nothing may still be running
     * on buffers the caller is about to reuse) */
    for (int s = 0; s < PF_STREAMS; s++) {
        LB_CU(c, lb_drv.EventRecord(ws->join[s], ws->stream[s]));
        LB_CU(c, lb_drv.StreamWaitEvent(main_stream, ws->join[s], 0));
    }
    if (st != LB_OK) return st == LB_ERR_CUDA ? lb_fail(c, LB_ERR_CUDA, "lb_model_prefill: a stream operation failed") : st;
    LB_CU(c, lb_drv.MemsetD32Async(m->d_pos, (unsigned)(pos0 + n - 1), 1, c->stream)); /* the sampling kernel advances it */
    LB_TRY(lb_dense_launch(c, m->lm_head, m->X, m->logits, m->vocab_s, H, LB_X_F32_RMSNORM, m->final_norm, cfg->eps, m->cand_val, m->cand_idx));
    LB_TRY(lb_model_launch_sampler(m));
    m->host_pos = pos0 + n;
    return next_out ? lb_model_read_next(m, next_out) : LB_OK;
}
