/* Host side of the persistent GEMV chain (kernels/chain.cu): the one-time strip packing of a
 * matrix, the checks, and the single launch.  The reference issues one launch_gemv per projection
 * (src/launcher.s:1226-1535); a chain replaces a run of them. */
#include "lb_internal.h"
#include "../kernels/params.h"

_Static_assert(sizeof(lb_chain_params) <= 4096, "kernel parameter block limit");
_Static_assert(LB_GEMV_CHAIN_MAX == LB_CHAIN_MAX_OPS, "public and kernel limits agree");

/* NULL when the chain kernel can run this shape on this GPU, else the reason */
static const char* chain_shape_problem(const lb_ctx* c, int K, int N, int swiglu) {
    if (K <= 0 || N <= 0 || K % LB_GEMV_GROUP != 0 || N % 32 != 0) return "needs K % 128 == 0 and N % 32 == 0";
    if (swiglu && N % 128 != 0) return "SwiGLU epilogue needs N % 128 == 0";
    const int upo = swiglu ? 2 : 1, units = N / 8 / upo, G = c->sm_count;
    const int most = (int)(((long long)units + G - 1) / G) * upo; /* octets of the widest strip */
    if (most > LB_CHAIN_MAX_OCTETS) return "more than 256 columns per SM";
    return NULL;
}

LB_API int lb_gemv_chain_supports(lb_ctx* c, int K, int N, int swiglu) {
    if (!c) return LB_ERR_INVALID;
    return chain_shape_problem(c, K, N, swiglu) ? LB_ERR_INVALID : LB_OK;
}

LB_API int lb_gemv_pack_version(void) { return LB_CHAIN_PACK_VERSION; }

LB_API size_t lb_gemv_packed_bytes(int K, int N) { return (size_t)(N / 8) * (size_t)(K / LB_GEMV_GROUP) * LB_CHAIN_RECORD; }

LB_API int lb_gemv_pack(lb_ctx* c, uint64_t qweight, uint64_t scales, uint64_t qzeros, int K, int N, int swiglu, uint64_t packed_out) {
    if (!c) return LB_ERR_INVALID;
    if (!qweight || !scales || !packed_out) return lb_fail(c, LB_ERR_INVALID, "lb_gemv_pack: NULL operand");
    const char* why = chain_shape_problem(c, K, N, swiglu);
    if (why) return lb_fail(c, LB_ERR_INVALID, "lb_gemv_pack: K=%d N=%d: %s", K, N, why);
    lb_pack_params p;
    memset(&p, 0, sizeof p);
    p.qweight = (const uint32_t*)qweight; p.scales = (const uint16_t*)scales; p.qzeros = (const uint32_t*)qzeros;
    p.out = (uint32_t*)packed_out;
    p.K = K; p.N = N; p.swiglu = swiglu ? 1 : 0; p.G = c->sm_count;
    void* params[] = {&p};
    LB_TRY(lb_launch(c, LBK_gemv_pack_strips, (unsigned)c->sm_count * 8, 1, 1, 256, 0, params, 0));
    /* remember the copy: lb_gemv_int4 on this qweight runs the strip-packed kernel from now on (until either buffer is freed) */
    int at = c->n_packed_reg;
    for (int i = 0; i < c->n_packed_reg; i++)
        if (c->packed_reg[i].qweight == qweight) at = i;
    if (at < LB_PACKED_REG_MAX) {
        c->packed_reg[at].qweight = qweight; c->packed_reg[at].packed = packed_out;
        c->packed_reg[at].K = K; c->packed_reg[at].N = N; c->packed_reg[at].swiglu = swiglu ? 1 : 0;
        if (at == c->n_packed_reg) c->n_packed_reg++;
    }
    return LB_OK;
}

/* internal: the packed copy of this matrix, or 0 */
uint64_t lb_packed_lookup(const lb_ctx* c, uint64_t qweight, int K, int N, int swiglu) {
    for (int i = 0; i < c->n_packed_reg; i++)
        if (c->packed_reg[i].qweight == qweight && c->packed_reg[i].K == K && c->packed_reg[i].N == N && c->packed_reg[i].swiglu == swiglu)
            return c->packed_reg[i].packed;
    return 0;
}

LB_API uint64_t lb_gemv_packed_copy(const lb_ctx* c, uint64_t qweight, int K, int N, int swiglu) {
    return c ? lb_packed_lookup(c, qweight, K, N, swiglu ? 1 : 0) : 0;
}

/* internal: a device buffer is going away */
void lb_packed_forget(lb_ctx* c, uint64_t ptr) {
    for (int i = 0; i < c->n_packed_reg;)
        if (c->packed_reg[i].qweight == ptr || c->packed_reg[i].packed == ptr) c->packed_reg[i] = c->packed_reg[--c->n_packed_reg];
        else i++;
}

/* Shared-memory plan of one chain launch: 0 ring slots = does not fit. */
typedef struct { int slots, table_rows, red_slots, tab_len; unsigned smem; } chain_plan;

static void chain_plan_make(const lb_ctx* c, const lb_chain_op* ops, int n_ops, chain_plan* pl) {
    int max_rows = 16, red_slots = 1, has_dn = 0;
    long long max_stages = 0; /* stages of the busiest CTA, all GEMVs of the chain */
    for (int i = 0; i < n_ops; i++) {
        const lb_chain_op* d = &ops[i];
        if (d->type != LB_CHAIN_OP_GEMV) { has_dn = 1; continue; }
        if (d->K / 8 > max_rows) max_rows = d->K / 8;
        const int widest = (int)(((long long)d->units + c->sm_count - 1) / c->sm_count) * d->upo;
        const int stages = ((widest + 1) / 2) * ((d->kg + LB_CHAIN_GC - 1) / LB_CHAIN_GC);
        if (stages > red_slots) red_slots = stages;
        max_stages += stages;
    }
    /* the activation table of the longest K, one 16-float slot of column sums per stage of a GEMV (the DeltaNet entries use
     * the same bytes: four units of 3232 B), the CTA's stage list, then as many ring slots per warp as fit, minus (when that
     * still leaves two slots) room for a small CTA of the neighbouring kernel */
    if (has_dn && red_slots < 13 * LB_CHAIN_WARPS) red_slots = 13 * LB_CHAIN_WARPS;
    const size_t table = (size_t)(max_rows / LB_GEMV_ROWS) * LB_CHAIN_GROUP_BYTES + 64;
    const int tab_len = (int)max_stages;
    const size_t fixed = table + (size_t)red_slots * 64 + (size_t)tab_len * 8 + 8;
    const size_t per_slot = (size_t)LB_CHAIN_WARPS * (LB_CHAIN_STAGE_BYTES + 8 + 4);
    const size_t limit = (size_t)c->max_smem_optin - (size_t)((c->fn_static_smem[LBK_gemv_chain] + 1023) & ~1023);
    int slots = limit > fixed + (size_t)c->chain_reserve ? (int)((limit - fixed - (size_t)c->chain_reserve) / per_slot) : 0;
    if (slots < 2) slots = limit > fixed ? (int)((limit - fixed) / per_slot) : 0;
    if (slots > 4) slots = 4;
    if (slots < 2) slots = 0;
    pl->slots = slots; pl->table_rows = max_rows; pl->red_slots = red_slots; pl->tab_len = tab_len;
    pl->smem = (unsigned)(fixed + (size_t)slots * per_slot);
}

/* internal: LB_OK when these entries can run as one launch */
int lb_chain_fits(lb_ctx* c, const lb_chain_op* ops, int n_ops) {
    if (n_ops < 1 || n_ops > LB_CHAIN_MAX_OPS) return LB_ERR_INVALID;
    chain_plan pl;
    chain_plan_make(c, ops, n_ops, &pl);
    return pl.slots ? LB_OK : LB_ERR_INVALID;
}

/* internal: launch kernel-level entries (GEMVs over packed weights, DeltaNet mixers) as one persistent kernel */
int lb_chain_launch(lb_ctx* c, const lb_chain_op* ops, int n_ops) {
    if (n_ops < 1 || n_ops > LB_CHAIN_MAX_OPS) return lb_fail(c, LB_ERR_INVALID, "chain: %d entries (1..%d)", n_ops, LB_CHAIN_MAX_OPS);
    lb_chain_params p;
    memset(&p, 0, sizeof p);
    memcpy(p.op, ops, sizeof(lb_chain_op) * (size_t)n_ops);
    chain_plan pl;
    chain_plan_make(c, ops, n_ops, &pl);
    if (!pl.slots) return lb_fail(c, LB_ERR_INVALID, "chain: %d entries (longest K %d) do not fit shared memory", n_ops, pl.table_rows * 8);
    /* GEMV fed by the GEMV right before it: hand the vector over through the producer's mailbox instead of a grid barrier */
    for (int i = 1; i < n_ops; i++) {
        lb_chain_op *a = &p.op[i - 1], *b = &p.op[i];
        if (!c->chain_mailbox || a->type != LB_CHAIN_OP_GEMV || b->type != LB_CHAIN_OP_GEMV || b->x != a->y) continue;
        /* without a barrier the consumer may read, besides the tagged vector, only what its own threads wrote before: an
         * accumulate target must have been written by the same column owners (same N) wherever this launch wrote it */
        int own = 1;
        if (b->y_mode == LB_Y_F32_ACCUM || b->y_mode == LB_Y_TP_ALLREDUCE)
            for (int j = 0; j < i; j++)
                if (p.op[j].type == LB_CHAIN_OP_GEMV && p.op[j].y == b->y && p.op[j].N != b->N) own = 0;
        if (!own) continue;
        const int f32_out = a->y_mode == LB_Y_F32 || a->y_mode == LB_Y_F32_ACCUM || a->y_mode == LB_Y_TP_ALLREDUCE;
        const int f16_out = a->y_mode == LB_Y_SWIGLU_F16;
        const int f32_in = b->x_mode == LB_X_F32 || b->x_mode == LB_X_F32_RMSNORM, f16_in = b->x_mode == LB_X_F16;
        if ((f32_out && f32_in && a->N == b->K && a->N <= LB_CHAIN_MAIL_WORDS) ||
            (f16_out && f16_in && a->N / 2 == b->K && a->N / 4 <= LB_CHAIN_MAIL_WORDS)) {
            a->mail = 1;
            b->x_src = i; /* index of the producer + 1 */
        }
    }
    /* per-head norm + gate prologue: the gate vector may be read (and its silu taken) before the entry's grid barrier when the
     * entry right before does not write it -- everything earlier in the launch is complete by then */
    for (int i = 0; i < n_ops; i++) {
        lb_chain_op* b = &p.op[i];
        if (b->type != LB_CHAIN_OP_GEMV || b->x_mode != LB_X_F32_HEADNORM_SILU) continue;
        const lb_chain_op* a = i ? &p.op[i - 1] : NULL;
        b->early_gate = !a || a->type == LB_CHAIN_OP_DELTANET || (a->type == LB_CHAIN_OP_GEMV && a->y != b->aux1 && (const void*)a->x_out != b->aux1);
    }
    p.mail = (unsigned long long*)c->chain_mail;
    p.slots = pl.slots;
    p.table_rows = pl.table_rows;
    p.red_slots = pl.red_slots;
    p.tab_len = pl.tab_len;
    p.n_ops = n_ops;
    p.trigger_op = n_ops - 1;
    p.status = (uint32_t*)c->dev_status;
    p.sync = (uint32_t*)c->gemv_counters; /* two words */
    p.timeline = (unsigned long long*)c->chain_timeline;
    void* params[] = {&p};
    return lb_launch(c, LBK_gemv_chain, (unsigned)c->sm_count, 1, 1, LB_CHAIN_THREADS, pl.smem, params, 1);
}

/* internal: fill a kernel-level GEMV entry; LB_ERR_INVALID (with the reason recorded) when the shape cannot run */
int lb_chain_fill_gemv(lb_ctx* c, lb_chain_op* d, const lb_gemv_op* o, int i) {
    if (!o->packed || !o->x || !o->y) return lb_fail(c, LB_ERR_INVALID, "GEMV chain[%d]: NULL operand", i);
    if (o->x_mode < LB_X_F16 || o->x_mode > LB_X_F32_HEADNORM_SILU || o->y_mode < LB_Y_F16 || o->y_mode > LB_Y_SWIGLU_F16)
        return lb_fail(c, LB_ERR_INVALID, "GEMV chain[%d]: unknown x_mode/y_mode %d/%d", i, o->x_mode, o->y_mode);
    if ((o->x_mode == LB_X_F32_RMSNORM && !o->aux0) || (o->x_mode == LB_X_F32_HEADNORM_SILU && (!o->aux0 || !o->aux1)))
        return lb_fail(c, LB_ERR_INVALID, "GEMV chain[%d]: norm prologue without its weight/gate operand", i);
    if (((o->packed | o->x | o->y | o->aux0 | o->aux1 | o->x_out) & 15ull) != 0)
        return lb_fail(c, LB_ERR_INVALID, "GEMV chain[%d]: operands must be 16-byte aligned", i);
    const int swiglu = o->y_mode == LB_Y_SWIGLU_F16;
    const char* why = chain_shape_problem(c, o->K, o->N, swiglu);
    if (why) return lb_fail(c, LB_ERR_INVALID, "GEMV chain[%d]: K=%d N=%d: %s", i, o->K, o->N, why);
    if (o->x_mode == LB_X_F32_HEADNORM_SILU && o->K > 8 * LB_CHAIN_THREADS * 2)
        return lb_fail(c, LB_ERR_INVALID, "GEMV chain[%d]: the per-head norm prologue takes K <= %d (K=%d)", i, 8 * LB_CHAIN_THREADS * 2, o->K);
    if (o->K > 8 * LB_CHAIN_THREADS * 5) return lb_fail(c, LB_ERR_INVALID, "GEMV chain[%d]: K=%d above %d", i, o->K, 8 * LB_CHAIN_THREADS * 5);
    memset(d, 0, sizeof *d);
    d->type = LB_CHAIN_OP_GEMV;
    d->packed = (const unsigned char*)o->packed;
    d->x = (const void*)o->x; d->y = (void*)o->y;
    d->aux0 = (const void*)o->aux0; d->aux1 = (const void*)o->aux1;
    d->x_out = (uint16_t*)o->x_out;
    d->K = o->K; d->N = o->N;
    d->kg = o->K / LB_GEMV_GROUP;
    d->upo = swiglu ? 2 : 1;
    d->units = o->N / 8 / d->upo;
    d->x_mode = o->x_mode; d->y_mode = o->y_mode;
    d->eps = o->eps;
    return LB_OK;
}

LB_API int lb_gemv_chain(lb_ctx* c, const lb_gemv_op* ops, int n_ops) {
    if (!c || !ops) return LB_ERR_INVALID;
    if (n_ops < 1 || n_ops > LB_CHAIN_MAX_OPS) return lb_fail(c, LB_ERR_INVALID, "GEMV chain: %d entries (1..%d)", n_ops, LB_CHAIN_MAX_OPS);
    lb_chain_op k[LB_CHAIN_MAX_OPS];
    for (int i = 0; i < n_ops; i++) LB_TRY(lb_chain_fill_gemv(c, &k[i], &ops[i], i));
    return lb_chain_launch(c, k, n_ops);
}
