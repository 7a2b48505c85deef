/* Private view of the decode-step model shared by lb_model.c (the step) and lb_prefill.c (the prompt pass). */
#ifndef LB_MODEL_PRIV_H
#define LB_MODEL_PRIV_H
#include "lb_internal.h"
#include "../kernels/params.h"

enum { /* src/launcher.s:92-141 */
    WS_DN_QKV = 0, WS_DN_Z = 3, WS_DN_OUT = 6, WS_DN_PROJ_A = 9, WS_DN_PROJ_B = 10, WS_DN_A_LOG = 11, WS_DN_DT_BIAS = 12,
    WS_DN_CONV1D = 13, WS_DN_NORM = 14,
    WS_FA_Q = 0, WS_FA_K = 3, WS_FA_V = 6, WS_FA_O = 9, WS_FA_Q_NORM = 12, WS_FA_K_NORM = 13,
    WS_GATE = 15, WS_UP = 18, WS_DOWN = 21, WS_INPUT_NORM = 24, WS_POST_NORM = 25,
    WG_EMBED = 0, WG_LM_HEAD = 1, WG_FINAL_NORM = 2
};

typedef struct {
    CUdeviceptr qweight, scales, qzeros; /* the reference format */
    CUdeviceptr packed;                  /* strip-packed copy for the persistent GEMV chain (0 = none) */
    int K, N;
} q4_mat;

typedef struct {
    int is_fa;
    q4_mat w_in, w_out, w_gateup, w_down;
    CUdeviceptr input_norm, post_norm;
    /* DeltaNet */
    CUdeviceptr proj_a, proj_b, a_log, dt_bias, conv_w, dn_norm, dn_state, conv_ring;
    CUdeviceptr snap_state, snap_conv; /* lb_model_checkpoint copies of dn_state and conv_ring (allocated on first use) */
    CUdeviceptr dn_params; /* lb_dn_layer_params of this layer in device memory, for the persistent chain */
    /* attention */
    CUdeviceptr q_norm, k_norm, k_cache, v_cache;
    int loaded;
} layer_t;

struct lb_model {
    lb_ctx* c;
    lb_model_cfg cfg;
    int tp_rank, tp_size;
    /* per-shard sizes */
    int HV, HK, HQ, HKV, inter_s; /* heads / intermediate columns on this shard */
    int C_s;                      /* conv channels on this shard: 2*HK*128 + HV*128 */
    layer_t* L;
    CUdeviceptr embed, lm_head, final_norm;
    int globals_loaded;
    /* activations */
    CUdeviceptr X, xn, in_out, mix_out, mlp_m, logits, d_token, d_pos, d_next, cand_val, cand_idx;
    int* h_next; /* pinned */
    int host_pos;  /* position the next step will decode, as the host knows it: set_input's value plus the steps issued since */
    uint64_t weight_bytes;
    lb_graph* graph;
    int step_kernels;
    lb_comm* comm;   /* tensor parallel: exchange buffers */
    int vocab_s;     /* vocabulary rows on this shard */
    int ar_count;    /* all-reduces issued so far in the step being built (slot parity) */
    int use_chain;   /* consecutive GEMVs of the step go out as one persistent launch (lb_gemv_chain) */
    CUdeviceptr tp_params[2]; /* tensor parallel: lb_tp_params of the two exchange slots in device memory, for the chain */
    lb_chain_op pend[LB_CHAIN_MAX_OPS]; /* GEMVs and DeltaNet mixers collected since the last stand-alone kernel */
    int n_pend;
    float temperature; int top_k; uint64_t sample_seed; /* top_k == 0: greedy (arg-max); else temperature / top-k sampling */
    struct lb_prefill_ws* ws; /* prompt-pass buffers (lb_prefill.c), NULL until the first prefill */
};


/* prompt-pass workspace (allocated by the first lb_model_prefill) */
typedef struct lb_prefill_ws lb_prefill_ws;

int lb_model_is_fa(const lb_model_cfg* c, int l);
int lb_model_launch_sampler(lb_model* m);
/* the decode-attention launch of one attention layer: inputs are the fused projection's fp32 row (per head 256 query then
 * 256 gate columns, then the key and value heads); pos_ptr != 0 reads the position from device memory (graph replay) */
int lb_model_launch_attention(lb_model* m, const layer_t* L, CUdeviceptr proj_row, CUdeviceptr out, CUdeviceptr pos_ptr, int pos, int splits_for);
#endif
