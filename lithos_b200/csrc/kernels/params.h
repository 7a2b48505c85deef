/* Kernel parameter blocks shared by the host layer (C) and the kernels (CUDA).
 * Every struct is passed by value as the single kernel parameter, so the
 * layout here IS the launch ABI of the primary entry points.  (The entry
 * points that keep the reference's own positional parameter blocks live under
 * csrc/compat/, one source per cubin, and do not use these structs.) */
#ifndef LB_KERNEL_PARAMS_H
#define LB_KERNEL_PARAMS_H
#include <stdint.h>

/* ---- int4 GEMV ---------------------------------------------------------- */
#define LB_GEMV_TILE_N 256   /* columns per CTA tile: eight 32-column TMA boxes */
#define LB_GEMV_GROUP 128    /* GPTQ group size along K */
#define LB_GEMV_ROWS 16      /* packed rows per group */
#define LB_GEMV_THREADS 160  /* 4 consumer warps (one 32-column box each) + 1 producer warp */
#define LB_GEMV_STAGE_BYTES 16384 /* one pipeline stage: 16 packed rows (one group) x 256 columns */

/* how the activation vector is produced from p.x */
enum {
    LB_X_F16 = 0,          /* x fp16 [K] */
    LB_X_F32 = 1,          /* x fp32 [K], rounded to fp16 */
    LB_X_F32_RMSNORM = 2,  /* x fp32 [K]; h = x*rsqrt(mean x^2+eps)*(1+w), w = aux0 bf16 [K] */
    LB_X_F32_HEADNORM_SILU = 3 /* x fp32 [K] in heads of 128; h = x*rsqrt(mean_head x^2+eps)*w[i]*silu(z),
                                  w = aux0 fp32 [128], z = aux1 fp32 [K] */
};
/* what is done with the N results */
enum {
    LB_Y_F16 = 0,       /* y fp16 [N] = result */
    LB_Y_F32 = 1,       /* y fp32 [N] = result */
    LB_Y_F32_ACCUM = 2, /* y fp32 [N] += result (residual add) */
    LB_Y_SWIGLU_F16 = 3, /* columns come in interleaved 64-wide blocks (gate block, up block, gate block, ...);
                           y fp16 [N/2] = silu(gate)*up */
    LB_Y_TP_ALLREDUCE = 4 /* persistent chain under tensor parallelism only: the fp32 results are this rank's partial sums of a
                           row-parallel projection; y (the residual stream) += their sum over all ranks, exchanged inside the
                           epilogue as (value, generation) words stored straight into every rank's buffer (ext = lb_tp_params) */
};

typedef struct {
    /* CUtensorMap over qweight viewed as [N/32][K/8][32] uint32: box 8 x 16 x 32, 128-byte swizzle */
    unsigned char tmap[128] __attribute__((aligned(64)));
    /* scales as fp16 [K/128, N], box = groups_per_split x 256; qzeros as u32 [K/128, N/8], box = groups_per_split x 32 */
    unsigned char tmap_sc[128] __attribute__((aligned(64)));
    unsigned char tmap_zr[128] __attribute__((aligned(64)));
    const uint32_t* qweight; /* [K/8, N] */
    const uint16_t* scales;  /* fp16 [K/128, N] */
    const uint32_t* qzeros;  /* [K/128, N/8] or NULL: zero-point 8 */
    const void* x;
    void* y;
    const void* aux0;
    const void* aux1;
    uint16_t* x_out;    /* optional fp16 [K]: the activation vector as the kernel used it */
    uint32_t* status;   /* device status word (bounded waits) */
    int32_t K, N;
    int32_t ksplit;           /* gridDim.y = cluster size along y */
    int32_t groups_per_split; /* ceil(K/128 / ksplit) */
    int32_t stages;           /* TMA ring depth */
    int32_t x_mode, y_mode;
    float eps;
} lb_gemv_params;

/* ---- chain of int4 GEMVs in ONE persistent launch (chain.cu) ------------------------------
 * One CTA per SM; CTA c owns a strip of whole columns of every GEMV (all of K), so no partial sums
 * cross CTAs.  The weights are read from a strip-packed copy made once by gemv_pack_strips:
 *   column unit = an octet of 8 columns (for the SwiGLU epilogue a unit is two octets: gate, up);
 *   CTA c owns octets [start(c), start(c+1)), start(c) = floor(c * units / G) * octets_per_unit,
 *   taken two at a time (a pair = the 16 rows of one tensor-core step; a strip with an odd number
 *   of octets ends with a single);
 *   per (octet, K-group) one 544-byte record
 *     [32 lanes x 16 B : lane (g = column in octet, t) holds the packed words of rows t, t+4, t+8, t+12 of the group]
 *     [8 x (fp16 scale, fp16 zero-point)];
 *   the strip is contiguous and pair-major: strip base = start(c) * KG * 544, then for every pair all
 *   K-groups in order, each group as [record of the first octet][record of the second octet].
 * A pipeline stage is LB_CHAIN_GC consecutive K-groups of one pair (4352 bytes), brought by one 1-D
 * bulk copy and consumed by ONE warp. */
#define LB_CHAIN_MAX_OPS 32
#define LB_CHAIN_PACK_VERSION 1      /* bumped whenever the strip-packed byte layout changes */
#define LB_CHAIN_OP_GEMV 0
#define LB_CHAIN_OP_DELTANET 1      /* the DeltaNet mixer of one layer (deltanet_core.cuh); ext = lb_dn_layer_params in device memory */

#define LB_CHAIN_WARPS 16            /* consumer warps; every warp streams its own stages */
#define LB_CHAIN_THREADS (LB_CHAIN_WARPS * 32)
#define LB_CHAIN_RECORD 544          /* bytes per (octet, K-group) */
#define LB_CHAIN_GC 4                /* K-groups per stage */
#define LB_CHAIN_STAGE_BYTES (LB_CHAIN_GC * 2 * LB_CHAIN_RECORD)
#define LB_CHAIN_MAX_OCTETS 32       /* octets one CTA may own */
#define LB_CHAIN_GROUP_BYTES 448     /* shared-memory bytes of one K-group's block of the activation table (chain.cu) */
#define LB_CHAIN_MAIL_WORDS 17408    /* 8-byte words of one entry's mailbox: fp32 results one per word, fp16 results two per word */

typedef struct {
    const unsigned char* packed; /* strip-packed weights (gemv_pack_strips) */
    const void* x;
    void* y;
    const void* aux0;
    const void* aux1;
    uint16_t* x_out;
    int32_t K, N;
    int32_t kg;       /* K / 128 */
    int32_t units;    /* column units: N/8 octets, or N/16 pairs for the SwiGLU epilogue */
    int32_t upo;      /* octets per unit: 1 or 2 */
    int32_t x_mode, y_mode;
    float eps;
    int32_t type;     /* LB_CHAIN_OP_* */
    int32_t early_gate; /* set by the launcher (LB_X_F32_HEADNORM_SILU): the entry right before this one does not write the gate
                           vector aux1, so its silu is taken before this entry's grid barrier */
    const void* ext;  /* parameters of a non-GEMV entry, in device memory */
    int32_t x_src;    /* set by the launcher: index + 1 of the entry of this launch whose tagged results are this GEMV's x
                         (then x is read from that entry's mailbox and NO grid barrier precedes this entry); 0 = read p.x */
    int32_t mail;     /* set by the launcher: this GEMV also publishes its results as (value, tag) words in its mailbox */
} lb_chain_op;

typedef struct {
    lb_chain_op op[LB_CHAIN_MAX_OPS];
    uint32_t* status;
    uint32_t* sync;       /* [0] grid-barrier arrivals, [1] CTAs that left; both zero between launches; [2] tag base, advanced
                             by LB_CHAIN_MAX_OPS per launch */
    int32_t n_ops;
    int32_t slots;        /* ring slots per warp */
    int32_t table_rows;   /* packed rows (K/8) the activation table holds: the largest K of the chain */
    int32_t red_slots;    /* 16-float slots for per-stage column sums: the most stages any CTA has in one GEMV of the chain */
    int32_t trigger_op;   /* griddepcontrol.launch_dependents is issued when this GEMV starts */
    int32_t tab_len;      /* entries of a CTA's stage list: the stages of the busiest CTA, all GEMVs of the chain */
    int32_t pad_[2];
    unsigned long long* mail; /* mailboxes: LB_CHAIN_MAX_OPS regions of LB_CHAIN_MAIL_WORDS 8-byte words (see chain.cu) */
    unsigned long long* timeline; /* optional [gridDim.x][LB_CHAIN_MAX_OPS][8] stamps of thread 0.  [0] %globaltimer (ns) when the entry
                                     is reached (the one stamp that compares across SMs); the rest are the SM's cycle counter:
                                     [1] entry reached, [2] grid barrier left, [3] input vector arrived, [4] activation table ready,
                                     [5] every stage of the strip consumed, [6] column sums ready, [7] entry finished (epilogue and,
                                     under tensor parallelism, the exchange); a mixer or all-reduce entry stamps [3..7] when it ends */
} lb_chain_params;

/* gemv_pack_strips: reference format -> strip-packed (one thread per 32-bit word of the output) */
typedef struct {
    const uint32_t* qweight; /* [K/8, N] */
    const uint16_t* scales;  /* fp16 [K/128, N] */
    const uint32_t* qzeros;  /* [K/128, N/8] or NULL: zero-point 8 */
    uint32_t* out;           /* N/8 * K/128 records of 136 words */
    int32_t K, N;
    int32_t swiglu;          /* input columns are interleaved 64-wide (gate, up) blocks; output units are (gate octet, up octet) pairs */
    int32_t G;               /* CTAs the strips are cut for */
} lb_pack_params;

/* ---- batched int4 projection: Y[B,N] = X[B,K] W ------------------------- */
typedef struct {
    /* gemm_int4_tc: CUtensorMap over X [B, K] fp16, box 64 k x NT tokens, 128-byte swizzle */
    unsigned char tmap_x[128] __attribute__((aligned(64)));
    const uint32_t* qweight; /* [K/8, N] */
    const uint16_t* scales;  /* fp16 [K/128, N] */
    const uint32_t* qzeros;  /* [K/128, N/8] or NULL: zero-point 8 */
    const uint16_t* x;       /* fp16 [B, K] */
    void* y;                 /* fp32 or fp16 [B, N] */
    int32_t K, N, B;
    int32_t y_f32;
    uint32_t* status; /* device status word for bounded waits (the host layer always passes the context's) */
    int32_t reserved;
} lb_bgemm_params;

/* ---- dense bf16 [N,K] x vector ------------------------------------------ */
typedef struct {
    const uint16_t* w; /* bf16 [N,K] row-major */
    const void* x;     /* fp16 or fp32 [K] */
    float* y;          /* fp32 [N] */
    const void* norm_w; /* bf16 [K] when x_mode == LB_X_F32_RMSNORM */
    int32_t N, K;
    int32_t x_mode; /* LB_X_F16 | LB_X_F32 | LB_X_F32_RMSNORM */
    float eps;
    float* part_val;  /* optional [gridDim.x]: largest y of the rows this CTA produced ... */
    int32_t* part_idx; /* ... and its row (smallest row on ties), for the greedy-sampling reduction */
    uint32_t* status;  /* device status word: set when a bounded wait for a weight row runs out (the rows left stay unwritten) */
} lb_dense_params;

/* ---- gated DeltaNet step -------------------------------------------------- */
typedef struct {
    float* state;      /* fp32 [HV,128,128] updated in place */
    const void* q;     /* [HK,128] bf16 or fp32 */
    const void* k;     /* [HK,128] */
    const void* v;     /* [HV,128] */
    const float* z;    /* fp32 [HV,128] or NULL: no silu(z) output gate */
    const float* g;    /* fp32 [HV] decay */
    const float* beta; /* fp32 [HV] */
    float* out;        /* fp32 [HV,128] */
    int32_t HV, HK;
} lb_deltanet_params;

typedef struct {
    const float* a;        /* [n] in_proj_a output */
    const float* a_log;    /* [n] */
    const float* dt_bias;  /* [n] */
    const float* b;        /* [n] in_proj_b output */
    float* g;              /* [n] decay out */
    float* beta;           /* [n] beta out */
    int32_t n;
} lb_decay_params;

/* ---- whole DeltaNet mixer of one layer (between the qkvz projection and the out projection) */
typedef struct {
    const float* qkvz;       /* fp32 [2*HK*128 + 2*HV*128]: q | k | v | z from the fused projection */
    const uint16_t* xn;      /* fp16 [hidden]: the normalised layer input (as the projection used it) */
    const uint16_t* proj_a;  /* bf16 [HV, hidden] in_proj_a */
    const uint16_t* proj_b;  /* bf16 [HV, hidden] in_proj_b */
    const float* a_log;      /* fp32 [HV] */
    const uint16_t* dt_bias; /* bf16 [HV] */
    const uint16_t* conv_w;  /* bf16 [4, C] planar, tap 0 = current token; C = 2*HK*128 + HV*128 */
    float* conv_ring;        /* fp32 [4, C]: slot (pos & 3) receives the current token's pre-conv values */
    float* state;            /* fp32 [HV,128,128] */
    float* out;              /* fp32 [HV,128] read-out (before the per-head norm and z gate) */
    const int* pos;          /* device int: position of the token being decoded */
    int32_t HV, HK, hidden;
    int32_t h0;              /* first global value head of this shard (tensor parallel), for nothing but clarity */
} lb_dn_layer_params;

/* ---- causal attention of a prompt chunk (pf_attn_prepare, pf_attn_chunk) --- */
typedef struct {
    const float* proj;        /* fp32 [T, ld]: per token, per head 256 query then 256 gate columns | k [HKV,256] | v [HKV,256] */
    const uint16_t* q_norm_w; /* bf16 [256] */
    const uint16_t* k_norm_w; /* bf16 [256] */
    uint16_t* k_cache;        /* bf16 [ctx,HKV,256]: rows pos0 .. pos0+T-1 are written by pf_attn_prepare */
    uint16_t* v_cache;
    uint16_t* qh;             /* bf16 [T,HQ,256]: the normalised, rotated, pre-scaled queries, leading term */
    uint16_t* ql;             /* bf16 [T,HQ,256]: what the rounding of qh left over */
    uint16_t* out;            /* fp16 [T,HQ,256]: attention output x sigmoid(gate), the o projection's input */
    int32_t ld, HQ, HKV, pos0, T, rot_dims;
    float eps;
    double rope_freq[64];     /* theta^(-i/(rot_dims/2)), computed on the host in double */
} lb_pf_attn_params;
/* pf_attn_chunk: query rows per CTA (16 per warp), threads, dynamic shared memory (two query tiles of ROWS x 528 B, two
 * stages of 32 K rows + 32 V rows x 528 B) */
#define LB_PF_ATTN_ROWS 32
#define LB_PF_ATTN_THREADS 64
#define LB_PF_ATTN_SMEM (2 * LB_PF_ATTN_ROWS * 528 + 2 * 2 * 32 * 528)

/* ---- GQA decode attention ------------------------------------------------- */
typedef struct {
    const void* q;        /* [HQ,256] bf16 or fp32 (raw, before norm) */
    const void* k_new;    /* [HKV,256] raw new key */
    const void* v_new;    /* [HKV,256] new value */
    const void* gate;     /* [HQ,256] or NULL */
    const uint16_t* q_norm_w; /* bf16 [256] or NULL: skip q/k norm */
    const uint16_t* k_norm_w; /* bf16 [256] */
    uint16_t* k_cache;    /* bf16 [ctx,HKV,256] */
    uint16_t* v_cache;
    float* out;           /* fp32 [HQ,256] */
    float* scratch;       /* split partials: [HKV][splits][G][(256 acc) + m + l] */
    uint32_t* counters;   /* one per kv head, zero between launches */
    const int* pos_ptr;   /* when non-NULL the position is read from device memory (graph replay) */
    int32_t pos;          /* position of the new token; rows [0,pos] are attended */
    int32_t HQ, HKV;
    int32_t splits;
    int32_t in_dtype;     /* 0 = bf16 inputs, 1 = fp32 inputs */
    int32_t gate_stride;  /* elements between consecutive heads of gate (256, or 512 when interleaved with q) */
    int32_t q_stride;     /* elements between consecutive heads of q */
    int32_t rot_dims;
    float rope_theta;
    float eps;
    double rope_freq[64]; /* theta^(-i/(rot_dims/2)), i < rot_dims/2 <= 64, computed on the host in double */
    uint32_t* status;     /* device status word for bounded waits (attn_decode_mma); may be NULL */
    int32_t coop;         /* attn_decode_mma: the grid fits the SMs one CTA each, so the CTAs of a KV head may wait for each
                             other and share the slice merge (counters[kv] arrivals, counters[8 + kv] finished) */
    int32_t max_ctx;      /* rows the caches hold (0 = not checked): a position outside [0, max_ctx) sets status
                             LB_DEV_POS_RANGE and the kernel returns without reading or writing a cache row */
} lb_attn_params;

/* ---- tensor-parallel exchange (comm.cu) ----------------------------------------------- */
#define LB_TP_MAX 8
/* Exchange buffer of one rank (every rank maps every peer's): float [2][size][n_max] partial vectors (slot = exchange
 * parity, then the rank that produced the vector), float [n_max] for the sampling record, the flag words, then
 * uint2 [2][size][n_max] (value, generation) words.
 * "Pull" exchanges (tp_allreduce_add): rank q leaves its partial in ITS OWN buffer at (slot, q),
 * raises flag [q] in every peer's flag array (system-scope release), readers load the vector from q's buffer.
 * "Pushed" exchanges (LB_Y_TP_ALLREDUCE): the thread that owns column n on rank q stores the 8-byte word (partial sum,
 * generation) into EVERY rank's word array at (slot, q, n) -- one store, delivered whole, so no fence and no flag -- and
 * then polls its own rank's array until the words of column n from all ranks carry this generation.  The same thread owns
 * column n on every rank (same matrix, same number of SMs), so nothing else has to be synchronised. */
typedef struct {
    float* x;                          /* residual stream [n] on this GPU */
    float* partials[LB_TP_MAX];        /* every rank's exchange buffer (peer pointers) */
    unsigned* peer_flags[LB_TP_MAX];   /* every rank's pull-flag array: unsigned [LB_TP_MAX] */
    unsigned* my_flags;                /* this rank's pull-flag array (local) */
    unsigned* gen;                     /* this rank's generation counter (local, advanced by the kernel) */
    unsigned* status;
    unsigned long long* words[LB_TP_MAX]; /* every rank's (value, generation) word array [2][size][n_max] (peer pointers) */
    int32_t n, n_max, slot, rank, size;
    int32_t pad_;
} lb_tp_params;
/* float offset of partial vector (slot, rank q) inside an exchange buffer; slot 2 is the sampling record */
#define LB_TP_PARTIAL(p, slot_, q) ((size_t)((slot_) == 2 ? 2 * (p).size : (slot_) * (p).size + (q)) * (size_t)(p).n_max)

typedef struct {
    lb_tp_params tp;        /* slot = 2: the record (logit, token) lives at the start of that slot */
    const float* cand_val;  /* this rank's per-CTA candidates from the LM-head kernel */
    const int32_t* cand_idx; /* rows inside this rank's vocabulary shard */
    int32_t n_cand, vocab_offset;
    int32_t* out_idx;
    int32_t* next_token;
    int32_t* pos;
} lb_tp_argmax_params;

#endif
