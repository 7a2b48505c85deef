/* liblithos_b200 — C ABI of the B200-native batch-1 decode hot path.
 *
 * Plain C: integer status codes, opaque context, device addresses as
 * uint64_t (CUdeviceptr), host buffers as plain pointers.  Each entry point
 * names the reference interface it replaces (paths relative to the reference
 * project root).  Every call returns LB_OK (0) or an error code; the text of
 * the last error is available from lb_last_error().  Nothing is ever skipped
 * silently: a missing kernel image, driver or GPU is an error, there is no CPU
 * fallback.
 *
 * Threading: one host thread per context, kernels are issued in program order
 * on the context's own stream (the reference launcher is single-threaded with
 * one main stream, src/launcher.s:455-492).
 */
#ifndef LITHOS_B200_H
#define LITHOS_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct lb_ctx lb_ctx;
typedef struct lb_model lb_model;

enum {
    LB_OK = 0,
    LB_ERR_INVALID = 1,     /* bad argument (shape, alignment, NULL) */
    LB_ERR_NO_DRIVER = 2,   /* libcuda.so.1 could not be loaded / no device */
    LB_ERR_CUDA = 3,        /* a CUDA driver call failed (see lb_last_error) */
    LB_ERR_NO_KERNEL = 4,   /* kernel image or entry point missing */
    LB_ERR_DEVICE_WAIT = 5, /* a bounded device-side wait gave up; status word in the message */
    LB_ERR_IO = 6,          /* file could not be read / bad weight index */
    LB_ERR_NOMEM = 7,
    LB_ERR_STATE = 8        /* call not valid in the current state (e.g. replay before capture) */
};

const char* lb_status_string(int status);
const char* lb_version(void);

/* ---- context ---------------------------------------------------------------
 * Replaces _start's cuInit / cuDeviceGet / cuCtxCreate / cuStreamCreate and
 * load_cubins (src/launcher.s:397-520, :3708-3965).  kernel_dir holds the
 * sm_100a cubins; NULL = the directory "kernels" beside the shared library.
 * Unlike the reference, a cubin or entry point that cannot be found is an
 * error here (the launcher stores NULL and skips every launch of it). */
int lb_init(int device, const char* kernel_dir, lb_ctx** out);
void lb_destroy(lb_ctx* ctx);
const char* lb_last_error(const lb_ctx* ctx);
int lb_device_sm_count(const lb_ctx* ctx);
/* status word written by bounded device-side waits (0 = none gave up); reading it synchronises the stream and,
 * when it is non-zero, returns LB_ERR_DEVICE_WAIT and clears the word.  The reference's own bounded wait traps the
 * GPU instead (runtime/sync.ls:50-60 sync_wait_flag_timeout); here the kernel returns and the host reads why:
 * 0x1001 a weight copy never landed, 0x1003 a peer GPU never published its flag, 0x1004 a CTA never reached the grid
 * barrier, 0x1005 the decode position lies outside the KV cache. */
int lb_device_status(lb_ctx* ctx, uint32_t* status_out);
int lb_reset_status(lb_ctx* ctx); /* clear the status word without reading it (stream-ordered) */
/* Time limit, in nanoseconds, of the kernels' waits on other CTAs and other GPUs (grid barrier, peer flags); 0 = the
 * built-in 2 s.  Stream-ordered: applies to kernels launched (or replayed) after it.  After a wait has run out, every
 * later wait returns at once until the status word is cleared, so a lost peer costs one limit, not one per exchange. */
int lb_set_wait_limit(lb_ctx* ctx, uint64_t ns);
/* number of kernels this library has launched on the context (graph replays count their kernel nodes) */
uint64_t lb_launch_count(const lb_ctx* ctx);
void lb_launch_count_reset(lb_ctx* ctx);
/* enable (1, default) / disable (0) programmatic dependent launch between consecutive kernels */
void lb_set_pdl(lb_ctx* ctx, int on);
/* bytes of an SM's shared memory lb_gemv_chain leaves free so that a CTA of the kernel before/after it can be
 * resident at the same time (default 32 KB; 0 = the deepest weight ring) */
void lb_set_chain_reserve(lb_ctx* ctx, int bytes);
/* on (default): where a GEMV of a chain reads the result vector of the GEMV right before it, the vector is handed over
 * as tagged 8-byte words that the consumer's loads wait on, and no grid barrier separates the two; off: a grid barrier
 * between every pair of entries.  Same results either way (the words carry the same fp32 / fp16 values). */
void lb_set_chain_mailbox(lb_ctx* ctx, int on);
/* Profiling hook: while buf != 0, every persistent-chain launch made (or captured) afterwards writes, for each SM and
 * chain entry, eight stamps of the SM's thread 0 into buf as u64 [SMs][LB_GEMV_CHAIN_MAX][8]: [0] %globaltimer (ns) when
 * the entry is reached, then the SM's cycle counter at [1] entry reached, [2] grid barrier left, [3] input vector arrived,
 * [4] activation table ready, [5] every weight stage consumed, [6] column sums ready, [7] entry finished (epilogue and,
 * under tensor parallelism, the exchange); a mixer entry stamps [3..7] when it ends.  Only [0] compares across SMs.
 * Launches overwrite each other's stamps. */
void lb_set_chain_timeline(lb_ctx* ctx, uint64_t buf);

/* ---- generic module load + launch ----------------------------------------------
 * The reference's own mechanism, kept as is: load_one_cubin = file read +
 * cuModuleLoadData + cuModuleGetFunction (src/launcher.s:3861-3965) and
 * cuLaunchKernel with a void** parameter array (src/launcher.s:744-762).  Any cubin
 * that keeps the reference's entry names and parameter blocks (the ones under
 * lithos_b200/kernels/compat do) can be driven through these three calls. */
int lb_module_load(lb_ctx* ctx, const char* cubin_path, int* module_out);
int lb_module_get_kernel(lb_ctx* ctx, int module, const char* entry, uint64_t* kernel_out);
int lb_launch_kernel(lb_ctx* ctx, uint64_t kernel, unsigned gx, unsigned gy, unsigned gz, unsigned bx, unsigned by,
                     unsigned bz, unsigned smem_bytes, void** params);

/* ---- CUDA graphs: whole sequences of launches as one submission ------------------
 * The reference issues ~1000 cuLaunchKernel calls per token (src/launcher.s:776-920) and
 * plans one submission per token (src/launcher.ls:16-106).  Everything launched through
 * this library between begin and end is captured (not run) and can then be replayed. */
typedef struct lb_graph lb_graph;
int lb_graph_begin_capture(lb_ctx* ctx);
int lb_graph_end_capture(lb_ctx* ctx, lb_graph** out);
int lb_graph_launch(lb_ctx* ctx, lb_graph* graph);
int lb_graph_kernel_count(const lb_graph* graph);
void lb_graph_destroy(lb_ctx* ctx, lb_graph* graph);

/* ---- device memory: replaces alloc_buffers (src/launcher.s:2981-3136) ------ */
int lb_malloc(lb_ctx* ctx, size_t bytes, uint64_t* dptr_out);
int lb_free(lb_ctx* ctx, uint64_t dptr);
int lb_malloc_host(lb_ctx* ctx, size_t bytes, void** host_out); /* pinned */
int lb_free_host(lb_ctx* ctx, void* host);
int lb_memcpy_h2d(lb_ctx* ctx, uint64_t dst, const void* src, size_t bytes); /* async on the context stream */
int lb_memcpy_d2h(lb_ctx* ctx, void* dst, uint64_t src, size_t bytes);       /* async on the context stream */
int lb_memcpy_d2d(lb_ctx* ctx, uint64_t dst, uint64_t src, size_t bytes);
int lb_memset(lb_ctx* ctx, uint64_t dst, int byte_value, size_t bytes);
int lb_sync(lb_ctx* ctx); /* replaces cuCtxSynchronize (src/launcher.s:931) */

/* ---- timing on the context's stream (CUDA events) -------------------------- */
int lb_timer_start(lb_ctx* ctx);
int lb_timer_stop(lb_ctx* ctx, float* ms_out); /* synchronises */
/* overwrite a > L2-sized buffer so that the next kernel starts with a cold L2 */
int lb_flush_l2(lb_ctx* ctx);

/* ---- seeded synthetic tensors (host) ---------------------------------------
 * Element i of stream s is a pure function of (seed, s, i). */
void lb_fill_u32(uint32_t* dst, size_t n, uint64_t seed, uint64_t stream); /* 8 nibbles U{0..15} per word */
void lb_fill_normal_f32(float* dst, size_t n, uint64_t seed, uint64_t stream, float mean, float std);
void lb_fill_normal_f16(uint16_t* dst, size_t n, uint64_t seed, uint64_t stream, float mean, float std);
void lb_fill_normal_bf16(uint16_t* dst, size_t n, uint64_t seed, uint64_t stream, float mean, float std);
void lb_fill_uniform_f32(float* dst, size_t n, uint64_t seed, uint64_t stream, float lo, float hi);
void lb_fill_scales_f16(uint16_t* dst, size_t n, uint64_t seed, uint64_t stream); /* |N(0,1)|*0.01+1e-3 */
void lb_convert_f32_to_f16(const float* src, uint16_t* dst, size_t n);
void lb_convert_f32_to_bf16(const float* src, uint16_t* dst, size_t n);
void lb_convert_f16_to_f32(const uint16_t* src, float* dst, size_t n);
void lb_convert_bf16_to_f32(const uint16_t* src, float* dst, size_t n);

/* ---- GPTQ int4 GEMV ----------------------------------------------------------
 * Replaces launch_proj + gptq_gemv_safe (src/launcher.s:1231-1535,
 * minds/gptq_gemv_safe.ptx:46-55; spec inference/gemv.ls:22-186).
 *   qweight int32 [K/8,N], scales fp16 [K/128,N], qzeros int32 [K/128,N/8]
 *   (0 = zero-point 8 as in every reference kernel).  K % 128 == 0, N % 32 == 0.
 * flags select the activation / result types (primary contract: fp16 x, fp16 y).
 * The result OVERWRITES y unless LB_GEMV_Y_ACCUM is set (the reference kernel
 * always accumulates into a caller-zeroed y).
 * Once lb_gemv_pack (below) has made a strip-packed copy of a matrix, lb_gemv_int4 on the same qweight pointer
 * (same K, N and SwiGLU flag) reads the copy and runs as a persistent chain of one: one CTA per SM owning whole
 * columns, no split-K and no cluster reduction.  Freeing either buffer with lb_free ends that. */
enum {
    LB_GEMV_X_F32 = 1 << 0,   /* x is fp32 (rounded to fp16 inside) instead of fp16 */
    LB_GEMV_Y_F32 = 1 << 1,   /* y is fp32 instead of fp16 */
    LB_GEMV_Y_ACCUM = 1 << 2, /* y (fp32) += result */
    LB_GEMV_Y_SWIGLU = 1 << 3 /* N columns are interleaved 64-wide (gate, up) blocks;
                                 y fp16 [N/2] = silu(gate)*up  (kernels.ls:61-66) */
};
int lb_gemv_int4(lb_ctx* ctx, uint64_t qweight, uint64_t scales, uint64_t qzeros, uint64_t x, uint64_t y, int K, int N,
                 int flags);
/* Same call with HOST buffers: copies the operands in, runs, copies y out, synchronises.
 * weights_resident != 0 reuses the device copy of the weights made by the previous call
 * with the same host pointers (only x goes in and y comes out). */
int lb_gemv_int4_host(lb_ctx* ctx, const uint32_t* qweight, const uint16_t* scales, const uint32_t* qzeros,
                      const void* x, void* y, int K, int N, int flags, int weights_resident);
/* fused variants used by the decode step (norm prologues): see lithos_b200/csrc/kernels/params.h */
int lb_gemv_int4_fused(lb_ctx* ctx, uint64_t qweight, uint64_t scales, uint64_t qzeros, uint64_t x, uint64_t y, int K,
                       int N, int x_mode, int y_mode, uint64_t aux0, uint64_t aux1, uint64_t x_out, float eps);
/* A chain of up to LB_GEMV_CHAIN_MAX fused GEMVs in ONE persistent launch (one CTA per SM, a grid
 * barrier between consecutive GEMVs): GEMV i+1 may read what GEMV i wrote.  Replaces a run of
 * consecutive launch_gemv calls of the decode step (src/launcher.s:829-933: out projection,
 * gate/up projection, down projection, next layer's input projections).  Same activation formats,
 * x_mode / y_mode values and results (to rounding) as lb_gemv_int4_fused called once per entry.
 * The weights are read from a strip-packed copy in which every SM's columns are contiguous:
 * lb_gemv_pack builds it once per matrix from the reference format (device to device;
 * lb_gemv_packed_bytes gives the size of the buffer the caller allocates; swiglu = 1 for a matrix
 * that will be used with the SwiGLU epilogue).  x and y of one entry must not overlap.
 * LB_ERR_INVALID when a shape puts more than 256 columns on one SM. */
#define LB_GEMV_CHAIN_MAX 32
typedef struct {
    uint64_t packed;                  /* from lb_gemv_pack */
    uint64_t x, y, aux0, aux1, x_out; /* as in lb_gemv_int4_fused */
    int32_t K, N, x_mode, y_mode;
    float eps;
    int32_t reserved;
} lb_gemv_op;
size_t lb_gemv_packed_bytes(int K, int N);
int lb_gemv_pack_version(void); /* version of the strip-packed byte layout (recorded beside measured DRAM traffic) */
int lb_gemv_pack(lb_ctx* ctx, uint64_t qweight, uint64_t scales, uint64_t qzeros, int K, int N, int swiglu, uint64_t packed_out);
/* the strip-packed copy lb_gemv_int4 would read for this matrix (made by lb_gemv_pack, neither buffer freed since), or 0 */
uint64_t lb_gemv_packed_copy(const lb_ctx* ctx, uint64_t qweight, int K, int N, int swiglu);
int lb_gemv_chain(lb_ctx* ctx, const lb_gemv_op* ops, int n_ops);
/* LB_OK when lb_gemv_pack / lb_gemv_chain accept this shape on this GPU (no launch) */
int lb_gemv_chain_supports(lb_ctx* ctx, int K, int N, int swiglu);
/* Batched projection: Y[B,N] = X[B,K] W for B = 1..LB_GEMM_MAX_BATCH tokens, W in the same three GPTQ
 * buffers as lb_gemv_int4 (read once for the whole batch), x fp16 [B,K] row-major, y fp32 [B,N]
 * (flags = LB_GEMV_Y_F32) or fp16 [B,N] (flags = 0).  K % 128 == 0, N % 16 == 0.
 * The reference's batched path is its prefill projection (kernels/projection_gemm.sass:390-631:
 * int4 -> fp16 dequantisation into shared memory, eight 16x8x16 tensor-core products per k-step);
 * One token is handed to the GEMV kernel of lb_gemv_int4.
 * 33..256 tokens run on the 5th-generation tensor cores (tcgen05.mma, accumulators in tensor memory):
 * the weights are dequantised to fp16 - (q - z) * s, q - z exact, one fp16 rounding for the scale - as the
 * reference kernel does, and handed to the tensor cores through tensor memory (129..256 tokens: one
 * product of 128 columns x 256 tokens per k step, the weights converted once for all of them).  Up to 32 tokens use mma.sync (faster there, measured):
 * q - z stays exact and the group scale multiplies the group's fp32 sum, so row b of Y equals
 * lb_gemv_int4 on row b of X to fp32 rounding.  LB_GEMM_TCGEN05 forces the tensor-memory kernel for
 * 9 tokens or more, LB_GEMM_MMA_SYNC the mma.sync kernels for every size up to 64 tokens (cross-checks).
 * Overwrites y.  x and y must not overlap. */
#define LB_GEMM_MMA_SYNC (1 << 4) /* flags: use the mma.sync kernels for every batch size */
#define LB_GEMM_TCGEN05 (1 << 5)  /* flags: use the tcgen05 kernel (B >= 9) */
#define LB_GEMM_MAX_BATCH 256
int lb_gemm_int4(lb_ctx* ctx, uint64_t qweight, uint64_t scales, uint64_t qzeros, uint64_t x_f16, uint64_t y, int K,
                 int N, int B, int flags);
/* bit-exact targets: W(k,n) = fma(float(q), s, -z*s) as fp32 [K,N]; q as u8 [K,N] */
int lb_gptq_dequant(lb_ctx* ctx, uint64_t qweight, uint64_t scales, uint64_t qzeros, uint64_t w_out_f32, int K, int N);
int lb_gptq_unpack(lb_ctx* ctx, uint64_t qweight, uint64_t q_out_u8, int K, int N);

/* ---- dense bf16 [N,K] x vector: replaces launch_lm_head (src/launcher.s:2903-2970) */
int lb_dense_bf16_gemv(lb_ctx* ctx, uint64_t w_bf16, uint64_t x, uint64_t y_f32, int N, int K, int x_is_f32);

/* ---- gated DeltaNet ------------------------------------------------------------
 * Replaces launch_recurrence / deltanet_fused (src/launcher.s:1960-2064,
 * inference/deltanet_fused.ls:37-151) and decay_gate + gate_sigmoid
 * (inference/decay_gate.ls:28-57, inference/recur.ls:45-55).
 * state fp32 [HV,128,128] in place; q,k [n_steps,HK,128]; v, z, out [n_steps,HV,128];
 * g, beta fp32 [n_steps,HV]; z == 0 skips the silu(z) gate.  in_is_f32 selects fp32
 * (else bf16) q/k/v.  n_steps > 1 runs consecutive tokens with the state held on chip. */
int lb_deltanet_step(lb_ctx* ctx, uint64_t state, uint64_t q, uint64_t k, uint64_t v, uint64_t z, uint64_t g,
                     uint64_t beta, uint64_t out, int HV, int HK, int n_steps, int in_is_f32);
int lb_decay_gate(lb_ctx* ctx, uint64_t a, uint64_t a_log, uint64_t dt_bias, uint64_t b, uint64_t g_out,
                  uint64_t beta_out, int n);

/* ---- GQA decode attention -----------------------------------------------------------
 * Replaces launch_rope + launch_kv_cache_write + launch_attention
 * (src/launcher.s:2260-2355, :2150-2247, :1846-1950; inference/attend.ls:21-191).
 * q [HQ,256], k_new/v_new [HKV,256], gate [HQ,256] (0 = none) in bf16 (or fp32 when
 * in_is_f32); q_norm_w/k_norm_w bf16 [256] (0 = no per-head RMSNorm); caches bf16
 * [ctx,HKV,256]; the new row is written at `pos`, rows [0,pos] are attended; out fp32. */
int lb_attention_decode(lb_ctx* ctx, uint64_t q, uint64_t k_new, uint64_t v_new, uint64_t gate, uint64_t q_norm_w,
                        uint64_t k_norm_w, uint64_t k_cache, uint64_t v_cache, uint64_t out, int pos, int HQ, int HKV,
                        int in_is_f32, int rot_dims, float rope_theta, float eps);

/* No counterpart in the reference.  The same decode-attention call for callers that cannot
 * allocate device memory and have no lb_ctx: code recording its own CUDA graph, a real-time loop
 * that sized everything at start-up, a plugin inside another runtime's memory pool, a process
 * held to a fixed memory budget.  The split-KV scratch is an array built into this library's
 * device image (798 976 bytes, held by every GPU that loads the library until the process exits),
 * so the call makes no cudaMalloc/cudaFree and uses no allocating library routine.
 *   - Runs on the CURRENT device, on `stream` (a CUstream / cudaStream_t, NULL = default stream).
 *   - Limits: at most 8 KV heads and 1, 2, 3, 4 or 6 query heads per KV head; the positions are
 *     cut into at most 16 slices whatever `pos` is.  Anything else returns LB_ERR_INVALID with
 *     the reason in `err`.
 *   - The first call on a device looks up the array's device address (cudaGetSymbolAddress) and
 *     sets the kernel's shared-memory limit; make that first call before any stream capture.
 *   - All calls on a device share the one array: calls that overlap on the GPU (two streams, two
 *     threads) race on it.  The call itself zeroes the arrival counters it needs on `stream`.
 * Arguments as lb_attention_decode; `err` (may be NULL) receives the error text. */
int lb_attention_decode_noalloc(void* stream, uint64_t q, uint64_t k_new, uint64_t v_new, uint64_t gate, uint64_t q_norm_w,
                                uint64_t k_norm_w, uint64_t k_cache, uint64_t v_cache, uint64_t out, int pos, int HQ,
                                int HKV, int in_is_f32, int rot_dims, float rope_theta, float eps, char* err, size_t errlen);

/* ---- small kernels ---------------------------------------------------------------------
 * rmsnorm: replaces launch_norm (src/launcher.s:1101-1219, inference/reduce.ls:21-147);
 * argmax: replaces the CPU argmax loop (src/launcher.s:962-1073, inference/reduce.ls:214-313);
 * embed: replaces the embed launch (src/launcher.s:713-762, inference/embed.ls:16-24). */
int lb_rmsnorm(lb_ctx* ctx, uint64_t x, uint64_t res, uint64_t w_bf16, uint64_t y, uint64_t sum_out, int rows, int D,
               float eps, int one_plus_w);
int lb_argmax(lb_ctx* ctx, uint64_t x_f32, int n, uint64_t out_idx_i32);
int lb_embed(lb_ctx* ctx, uint64_t table_bf16, uint64_t token_i32, uint64_t out_f32, int D);
/* Temperature + top-k sampling: what the reference's `sample` kernel is specified to do (kernels/README.md:104-117: "top-k
 * sampling ... with temperature scaling"; its shipped code only takes the arg-max, which compat/sample.cubin reproduces).
 * Among the top_k (1..64) largest logits -- ties by smaller index -- p_i = softmax(l_i / temperature); the token is the
 * first whose cumulative probability exceeds u, where u is element `counter` of stream 7777 of the seeded generator
 * (lb_fill_uniform_f32(.., seed, 7777, 0, 1)).  probs_out (fp32 [top_k]) and idx_out (i32 [top_k]) may be 0. */
int lb_sample_topk(lb_ctx* ctx, uint64_t logits_f32, int n, float temperature, int top_k, uint64_t seed, uint64_t counter,
                   uint64_t out_idx_i32, uint64_t probs_out, uint64_t idx_out);

/* ---- tensor-parallel exchange buffers (no counterpart in the reference: it is single-GPU) ---
 * One process per GPU.  Each rank creates its buffer, the launcher passes the 64-byte IPC
 * handles around (any transport), every rank opens its peers.  The exchange kernels use plain
 * peer loads/stores over NVLink with bounded waits. */
typedef struct lb_comm lb_comm;
int lb_comm_create(lb_ctx* ctx, int rank, int size, int n_max, lb_comm** out); /* n_max >= hidden size */
int lb_comm_rank(const lb_comm* comm);
int lb_comm_size(const lb_comm* comm);
int lb_comm_handle(lb_comm* comm, void* handle_out64);
int lb_comm_open(lb_comm* comm, const void* handles_size_x_64);
/* A peer whose buffer this process can address directly (a second GPU of the same process with peer access enabled):
 * its lb_comm_buffer, lb_comm_bytes long, instead of an IPC handle. */
int lb_comm_set_peer(lb_comm* comm, int rank, uint64_t peer_buffer);
uint64_t lb_comm_buffer(const lb_comm* comm);      /* this rank's exchange buffer: float [2][size][n_max] partial vectors, a sampling record, then the flags */
size_t lb_comm_bytes(const lb_comm* comm);
size_t lb_comm_partial_offset(const lb_comm* comm, int slot, int rank); /* byte offset of rank's partial vector of slot 0 / 1 */
size_t lb_comm_flags_offset(const lb_comm* comm);  /* byte offset of the flag array u32 [8] (one generation word per rank) */
/* One exchange outside the decode step: x[0..n) += the sum over ranks, in rank order, of the partial vectors every
 * rank has left at lb_comm_partial_offset(slot, its rank) of its own buffer.  Bounded: a rank that never publishes makes the kernel return with
 * status 0x1003 after the wait limit. */
int lb_comm_allreduce(lb_comm* comm, uint64_t x_f32, int n, int slot);
void lb_comm_destroy(lb_comm* comm);

/* ---- the whole decode step ------------------------------------------------------------
 * Replaces decode_one_token and its launch_* helpers (src/launcher.s:685-1092), the per-layer
 * weight-slot table (src/launcher.s:92-141, 298-311) and the buffer plan (src/launcher.s:143-169).
 * Layer l is a full-attention layer when l % fa_period == fa_period-1, otherwise a Gated
 * DeltaNet layer (compiler/megakernel-link.ls:204-211); both are followed by the SwiGLU MLP. */
typedef struct {
    int32_t n_layers, hidden, inter, vocab;
    int32_t dn_k_heads, dn_v_heads, dn_dim, conv_taps; /* dn_dim must be 128, conv_taps 4 */
    int32_t fa_q_heads, fa_kv_heads, fa_dim, rot_dims; /* fa_dim must be 256 */
    int32_t group, fa_period, max_ctx, reserved;       /* group must be 128 */
    float eps, rope_theta;
} lb_model_cfg;

enum { LB_WS_SLOTS = 26, LB_WG_SLOTS = 3 }; /* slot indices as in src/launcher.s:92-141 and :306-311 */

/* tp_rank / tp_size: tensor-parallel shard held by this context (1 GPU: 0 / 1). */
int lb_model_create(lb_ctx* ctx, const lb_model_cfg* cfg, int tp_rank, int tp_size, lb_model** out);
/* tensor parallel: the exchange buffers (all peers opened) this model's all-reduces go through */
/* on (default): consecutive projections of the step are issued as one persistent launch (lb_gemv_chain);
 * off: one launch per projection.  Takes effect at the next lb_model_decode / lb_model_capture. */
int lb_model_set_chain(lb_model* m, int on);
int lb_model_set_comm(lb_model* m, lb_comm* comm);
void lb_model_destroy(lb_model* m);
/* Host tensors of one layer in the reference's slot order (26 pointers, unused slots NULL) in
 * the reference's packed formats; they are re-laid (projections that share an input fused along
 * N, gate/up interleaved, tensor-parallel shard cut out) and uploaded.  Replaces load_weights
 * (src/launcher.s:3284-3683). */
int lb_model_load_layer(lb_model* m, int layer, const void* const* slots);
int lb_model_load_globals(lb_model* m, const void* const* globals); /* embed, lm_head, final_norm */
const lb_model_cfg* lb_model_config(const lb_model* m);

/* ---- weight_index.bin: the launcher's weight-table file (src/launcher.s:3267-3282 format, :3284-3683 load_weights) ----
 * <model_dir>/weight_index.bin names the shard files and gives (shard, offset, size) for 26 slots per layer + 3
 * globals; load_weights maps the shards and resolves the pointers.  lb_load_weights does the same and hands every
 * layer to lb_model_load_layer.  Unlike the launcher (which prints a message and goes on with NULL pointers), a bad
 * magic or version, a truncated index, a shard index out of range, an entry that runs past its shard or does not
 * have the size the model shape implies are LB_ERR_IO, a missing required slot LB_ERR_INVALID.
 * The host-only calls (open / entry / check / close, lb_save_weights) need no GPU; `err` receives the reason. */
typedef struct lb_weight_index lb_weight_index;
int lb_weight_index_open(const char* model_dir, lb_weight_index** out, char* err, size_t errlen);
int lb_weight_index_dims(const lb_weight_index* w, int* n_layers, int* n_slots, int* n_globals, int* n_shards);
/* host pointer into the mapped shard and size of (layer, slot); layer < 0 addresses global `slot`; unused -> NULL, 0 */
int lb_weight_index_entry(const lb_weight_index* w, int layer, int slot, const void** ptr, size_t* bytes);
int lb_weight_index_check(const lb_weight_index* w, const lb_model_cfg* cfg, char* err, size_t errlen);
void lb_weight_index_close(lb_weight_index* w);
/* bytes of slot `slot` of `layer` / of global `which` for this model shape (0 = unused in that kind of layer):
 * int4 tensors in the reference's packing, norm / conv / projection-a,b tensors bf16, A_log and the per-head norm fp32 */
size_t lb_model_slot_bytes(const lb_model_cfg* cfg, int layer, int slot);
size_t lb_model_global_bytes(const lb_model_cfg* cfg, int which);
/* Writes <model_dir>/weight_index.bin and one raw shard file holding the given host tensors (layer_slots is
 * [n_layers * 26], unused slots NULL).  Stands in for the reference's gen_weight_index.py, which is not in its tree. */
int lb_save_weights(const char* model_dir, const lb_model_cfg* cfg, const void* const* layer_slots, const void* const* globals,
                    char* err, size_t errlen);
int lb_load_weights(lb_ctx* ctx, const char* model_dir, lb_model* m);
/* Writes <model_dir>/weight_index.bin for a safetensors checkpoint lying in model_dir: every *.safetensors file becomes a
 * shard (name order), every slot the (shard, file offset, size) of the tensor the reference resolves it from
 * (model.layers.<n>.<suffix> with the suffixes of src/launcher.s:92-141, compiler/megakernel-link.ls:220-269; globals
 * model.embed_tokens.weight, lm_head.weight, model.norm.weight, :825-827), so that lb_load_weights -- or the reference's
 * launcher -- reads the checkpoint in place.  Host only.  A tensor that is missing is LB_ERR_INVALID, one whose byte size is
 * not what the model shape implies, or a malformed header, LB_ERR_IO.  The tensors are taken as stored: AutoGPTQ's
 * "zero-point minus one" convention, where a checkpoint uses it, is the exporter's to undo. */
int lb_weight_index_from_safetensors(const char* model_dir, const lb_model_cfg* cfg, char* err, size_t errlen);
/* Host-only view of the same re-layout (no GPU needed): device matrix `which` (0 fused input
 * projections, 1 out/o projection, 2 gate|up interleaved, 3 down) of tensor-parallel shard
 * tp_rank/tp_size for `layer`.  Call with NULL outputs for the sizes, then with buffers of
 * K/8*N, K/128*N and K/128*N/8 elements. */
int lb_model_shard_host(const lb_model_cfg* cfg, int tp_rank, int tp_size, int layer, int which, const void* const* slots,
                        uint32_t* qweight_out, uint16_t* scales_out, uint32_t* qzeros_out, int* K_out, int* N_out);
/* Seeded synthetic weights with the shapes/distributions of the benchmark definition; tensor
 * (layer, slot) is stream (layer+1)*100+slot of the generator, globals are streams 1..3. */
int lb_model_fill_synthetic(lb_model* m, uint64_t seed);
int lb_model_reset_state(lb_model* m); /* zero DeltaNet states, conv history and KV caches */
/* device address of a layer's recurrent buffers: which = 0 DeltaNet state / K cache,
 * 1 conv ring [4][C] (slot = position & 3) / V cache */
int lb_model_state_ptr(lb_model* m, int layer, int which, uint64_t* dptr_out, size_t* bytes_out);
/* Snapshot / restore of the recurrent state (every DeltaNet layer's state matrix and convolution history), for
 * speculative decoding: decode ahead, then lb_model_rollback and continue from the checkpointed position.
 * Replaces the reference's state_rollback copy kernel (inference/recur.ls:82-86, kernels/recurrence_rollback.sass).
 * Stream-ordered device-to-device copies; the KV caches are not copied (rows past the position are never read).
 * LB_ERR_STATE from lb_model_rollback when no checkpoint was taken. */
int lb_model_checkpoint(lb_model* m);
int lb_model_rollback(lb_model* m);

int lb_model_logits_ptr(lb_model* m, uint64_t* dptr_out);
uint64_t lb_model_weight_bytes(const lb_model* m); /* bytes of weights one decode step streams on this shard */
/* One token, launch by launch: token and position go in, the greedy next token comes out. */
int lb_model_decode(lb_model* m, int token, int pos, int* next_out);
/* Capture the whole step once; then each replay consumes the token/position left on the device
 * by the previous step (set them with lb_model_set_input) and leaves the next token there. */
int lb_model_capture(lb_model* m);
int lb_model_set_input(lb_model* m, int token, int pos); /* stream-ordered, by value: safe to call back to back */
/* n graph launches, no host round trip.  LB_ERR_INVALID (nothing launched) when the steps would run past max_ctx:
 * the host tracks the position from lb_model_set_input / lb_model_decode plus the steps issued since. */
int lb_model_replay(lb_model* m, int n_steps);
int lb_model_read_next(lb_model* m, int* next_out);   /* synchronises */
/* The prompt pass.  Runs tokens[0..n) at positions pos0 .. pos0+n-1 through the model in chunks of up to 256 and leaves
 * the state a token-by-token lb_model_decode of the same tokens leaves (DeltaNet states, convolution rings, KV rows);
 * *next_out (may be NULL) receives the greedy token that follows the prompt, the logits of the last prompt token are
 * in lb_model_logits_ptr, and lb_model_replay / lb_model_decode continue from position pos0+n.  Every projection of a
 * chunk is one lb_gemm_int4 call (the reference's prompt path is its dequantising tensor-core GEMM,
 * kernels/projection_gemm.sass:390-631; layer order compiler/megakernel-link.ls:281-525), the recurrence keeps the state
 * on chip for the chunk, attention is one causal tensor-core kernel per chunk.  Up to four chunks are in flight on
 * streams of the library's own (a layer of a chunk waits for the same layer of the chunk before it); they start behind
 * what the context's stream holds when the call is made and the context's stream continues behind them.  The first call
 * allocates the chunks' buffers (about 90 MB each at the 27B widths).  Single GPU (tp_size 1) only. */
int lb_model_prefill(lb_model* m, const int* tokens, int n, int pos0, int* next_out);
int lb_model_step_kernels(const lb_model* m);         /* kernels per decode step */
/* top_k == 0 (default): greedy; else every step samples among the top_k largest logits at `temperature`, the draw being a
 * function of (seed, position).  Takes effect at the next lb_model_decode / lb_model_capture.  Single GPU only. */
int lb_model_set_sampling(lb_model* m, float temperature, int top_k, uint64_t seed);
/* The launcher's decode loop (src/launcher.s:552-652, :931-1087): run the prompt (lb_model_prefill), then decode until
 * `eos` (248044 for the reference model; negative = none), max_new tokens or a full context.  out [max_new] receives
 * the generated tokens, *n_out their number. */
int lb_model_generate(lb_model* m, const int* prompt, int n_prompt, int max_new, int eos, int* out, int* n_out);

#ifdef __cplusplus
}
#endif
#endif
