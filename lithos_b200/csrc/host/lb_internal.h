/* Internal declarations shared by the host-side C files of liblithos_b200. */
#ifndef LB_INTERNAL_H
#define LB_INTERNAL_H

#include <stddef.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <cuda.h> /* types and enums only: the driver itself is bound at run time */

#include "lithos_b200.h"

#define LB_API __attribute__((visibility("default")))

/* ---- run-time binding of the CUDA driver (libcuda.so.1) ---------------- */
/* The library must load (and export its symbols) on a machine without a GPU
 * driver, so nothing links against libcuda: entry points are fetched through
 * cuGetProcAddress on first lb_init. */
#define LB_DRIVER_FUNCS(X)                                                                                      \
    X(Init, cuInit, (unsigned int))                                                                             \
    X(DriverGetVersion, cuDriverGetVersion, (int*))                                                             \
    X(DeviceGet, cuDeviceGet, (CUdevice*, int))                                                                 \
    X(DeviceGetCount, cuDeviceGetCount, (int*))                                                                 \
    X(DeviceGetAttribute, cuDeviceGetAttribute, (int*, CUdevice_attribute, CUdevice))                           \
    X(DevicePrimaryCtxRetain, cuDevicePrimaryCtxRetain, (CUcontext*, CUdevice))                                 \
    X(DevicePrimaryCtxRelease, cuDevicePrimaryCtxRelease, (CUdevice))                                           \
    X(CtxSetCurrent, cuCtxSetCurrent, (CUcontext))                                                              \
    X(CtxSynchronize, cuCtxSynchronize, (void))                                                                 \
    X(MemAlloc, cuMemAlloc, (CUdeviceptr*, size_t))                                                             \
    X(MemFree, cuMemFree, (CUdeviceptr))                                                                        \
    X(MemHostAlloc, cuMemHostAlloc, (void**, size_t, unsigned int))                                             \
    X(MemFreeHost, cuMemFreeHost, (void*))                                                                      \
    X(MemcpyHtoDAsync, cuMemcpyHtoDAsync, (CUdeviceptr, const void*, size_t, CUstream))                         \
    X(MemcpyDtoHAsync, cuMemcpyDtoHAsync, (void*, CUdeviceptr, size_t, CUstream))                               \
    X(MemcpyDtoDAsync, cuMemcpyDtoDAsync, (CUdeviceptr, CUdeviceptr, size_t, CUstream))                         \
    X(MemsetD8Async, cuMemsetD8Async, (CUdeviceptr, unsigned char, size_t, CUstream))                           \
    X(MemsetD32Async, cuMemsetD32Async, (CUdeviceptr, unsigned int, size_t, CUstream))                          \
    X(ModuleLoadData, cuModuleLoadData, (CUmodule*, const void*))                                               \
    X(ModuleUnload, cuModuleUnload, (CUmodule))                                                                 \
    X(ModuleGetFunction, cuModuleGetFunction, (CUfunction*, CUmodule, const char*))                             \
    X(FuncSetAttribute, cuFuncSetAttribute, (CUfunction, CUfunction_attribute, int))                            \
    X(FuncGetAttribute, cuFuncGetAttribute, (int*, CUfunction_attribute, CUfunction))                           \
    X(LaunchKernel, cuLaunchKernel,                                                                             \
      (CUfunction, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, CUstream, void**, void**)) \
    X(LaunchKernelEx, cuLaunchKernelEx, (const CUlaunchConfig*, CUfunction, void**, void**))                    \
    X(StreamCreate, cuStreamCreate, (CUstream*, unsigned int))                                                  \
    X(StreamDestroy, cuStreamDestroy, (CUstream))                                                               \
    X(StreamSynchronize, cuStreamSynchronize, (CUstream))                                                       \
    X(EventCreate, cuEventCreate, (CUevent*, unsigned int))                                                     \
    X(EventDestroy, cuEventDestroy, (CUevent))                                                                  \
    X(EventRecord, cuEventRecord, (CUevent, CUstream))                                                          \
    X(StreamWaitEvent, cuStreamWaitEvent, (CUstream, CUevent, unsigned int))                                    \
    X(EventSynchronize, cuEventSynchronize, (CUevent))                                                          \
    X(EventElapsedTime, cuEventElapsedTime, (float*, CUevent, CUevent))                                         \
    X(StreamBeginCapture, cuStreamBeginCapture, (CUstream, CUstreamCaptureMode))                                \
    X(StreamEndCapture, cuStreamEndCapture, (CUstream, CUgraph*))                                               \
    X(GraphInstantiate, cuGraphInstantiateWithFlags, (CUgraphExec*, CUgraph, unsigned long long))                        \
    X(GraphLaunch, cuGraphLaunch, (CUgraphExec, CUstream))                                                      \
    X(GraphDestroy, cuGraphDestroy, (CUgraph))                                                                  \
    X(GraphExecDestroy, cuGraphExecDestroy, (CUgraphExec))                                                      \
    X(GraphGetNodes, cuGraphGetNodes, (CUgraph, CUgraphNode*, size_t*))                                         \
    X(IpcGetMemHandle, cuIpcGetMemHandle, (CUipcMemHandle*, CUdeviceptr))                                       \
    X(IpcOpenMemHandle, cuIpcOpenMemHandle, (CUdeviceptr*, CUipcMemHandle, unsigned int))                       \
    X(IpcCloseMemHandle, cuIpcCloseMemHandle, (CUdeviceptr))                                                    \
    X(TensorMapEncodeTiled, cuTensorMapEncodeTiled,                                                             \
      (CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*, \
       const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill)) \
    X(GetErrorString, cuGetErrorString, (CUresult, const char**))                                               \
    X(GetErrorName, cuGetErrorName, (CUresult, const char**))

typedef struct {
#define X(field, sym, args) CUresult(CUDAAPI* field) args;
    LB_DRIVER_FUNCS(X)
#undef X
    int loaded;
} lb_driver;

extern lb_driver lb_drv;
int lb_driver_load(char* err, size_t errlen); /* LB_OK or LB_ERR_NO_DRIVER */

/* ---- kernels (entry points inside the cubins) -------------------------- */
#define LB_KERNELS(X)                 \
    X(gemv_int4_w256)                 \
    X(gemv_chain)                     \
    X(gemv_pack_strips)               \
    X(gemm_int4_mma_b8)               \
    X(gemm_int4_mma_b16)              \
    X(gemm_int4_mma_b32)              \
    X(gemm_int4_mma_b64)              \
    X(gemm_int4_tc)                   \
    X(gemm_int4_tc_g1)                \
    X(gemm_int4_tc_ta)                \
    X(gemm_int4_tc_ta_g1)             \
    X(gptq_dequant_f32)               \
    X(gptq_unpack_u8)                 \
    X(dense_bf16_gemv)                \
    X(dense_bf16_stream)              \
    X(decay_gate_beta)                \
    X(deltanet_step_bf16)             \
    X(deltanet_step_f32)              \
    X(deltanet_layer_fused)           \
    X(attn_decode_split)              \
    X(attn_decode_mma)                \
    X(embed_bf16)                     \
    X(argmax_f32)                     \
    X(topk_sample_f32)                \
    X(rmsnorm_f32)                    \
    X(tp_allreduce_add)               \
    X(tp_argmax_exchange)             \
    X(pf_embed)                       \
    X(pf_rmsnorm_f16)                 \
    X(pf_dn_frontend)                 \
    X(pf_dn_ring)                     \
    X(pf_ab_gate)                     \
    X(pf_headnorm_gate_f16)           \
    X(pf_swiglu_f16)                  \
    X(pf_add)                         \
    X(pf_attn_prepare)                \
    X(pf_attn_chunk)                  \
    X(l2_flush)

enum {
#define X(name) LBK_##name,
    LB_KERNELS(X)
#undef X
    LBK_COUNT
};

#define LB_MAX_MODULES 64
#define LB_MAX_PEERS 8

#define LB_PACKED_REG_MAX 1024
struct lb_ctx {
    int device;
    CUdevice cu_dev;
    CUcontext cu_ctx;
    CUstream stream;
    CUevent ev[2];
    int sm_count;
    int max_smem_optin;
    CUmodule modules[LB_MAX_MODULES];
    int n_modules;
    CUfunction fn[LBK_COUNT];
    int fn_static_smem[LBK_COUNT]; /* static shared memory of each kernel, bytes */
    /* split-K scratch shared by every GEMV launched on this context's stream */
    CUdeviceptr gemv_partial; /* fp32 [LB_GEMV_MAX_SPLITS][LB_GEMV_SCRATCH_N] */
    CUdeviceptr gemv_counters; /* u32 per column tile, self-resetting */
    CUdeviceptr attn_scratch;  /* split-KV partials */
    size_t attn_scratch_bytes;
    CUdeviceptr dev_status; /* u32 words written by bounded device-side waits */
    CUdeviceptr flush_buf;  /* L2 flush target */
    size_t flush_bytes;
    uint64_t launches; /* kernels launched (or graph nodes replayed) since reset */
    int pdl;           /* use programmatic dependent launch between kernels */
    CUdeviceptr chain_timeline; /* optional time-stamp buffer handed to every chain launch (lb_set_chain_timeline) */
    int chain_reserve; /* bytes of an SM's shared memory the GEMV chain leaves to a neighbouring kernel's CTA */
    CUdeviceptr chain_mail; /* mailboxes of the persistent chain: LB_CHAIN_MAX_OPS x LB_CHAIN_MAIL_WORDS 8-byte (value, tag) words */
    /* strip-packed copies made by lb_gemv_pack and still alive: lb_gemv_int4 runs the strip-packed kernel for these matrices */
    struct { uint64_t qweight, packed; int K, N, swiglu; } packed_reg[LB_PACKED_REG_MAX];
    int n_packed_reg;
    int chain_mailbox;      /* hand vectors from a GEMV to the next one through the mailbox (1, default) or a grid barrier (0) */
    int capturing;     /* stream capture in progress */
    uint64_t capture_launches0;
    char err[512];
};

#define LB_GEMV_SCRATCH_N (1 << 18) /* widest N a split-K GEMV may have */
#define LB_GEMV_MAX_SPLITS 8 /* = the portable thread-block-cluster size */

int lb_fail(lb_ctx* c, int status, const char* fmt, ...);

int lb_cu(lb_ctx* c, CUresult r, const char* what);
#define LB_CU(c, call)                                  \
    do {                                                \
        int _s = lb_cu((c), (call), #call);             \
        if (_s != LB_OK) return _s;                     \
    } while (0)
#define LB_TRY(expr)                  \
    do {                              \
        int _s = (expr);              \
        if (_s != LB_OK) return _s;   \
    } while (0)

int lb_launch(lb_ctx* c, int kernel, unsigned gx, unsigned gy, unsigned gz, unsigned bx, unsigned smem, void** params,
              int pdl);
int lb_launch_cluster(lb_ctx* c, int kernel, unsigned gx, unsigned gy, unsigned gz, unsigned bx, unsigned smem,
                      void** params, int pdl, unsigned cluster_y);

/* rng helpers used by the synthetic model builder */
uint64_t lb_rng_u64(uint64_t seed, uint64_t stream, uint64_t i);
uint64_t lb_packed_lookup(const lb_ctx* c, uint64_t qweight, int K, int N, int swiglu); /* lb_chain.c: strip-packed copy of a matrix, or 0 */
void lb_packed_forget(lb_ctx* c, uint64_t ptr);                                         /* a device buffer is going away */
uint32_t lb_rng_word(uint64_t seed, uint64_t stream, uint64_t i);
uint16_t lb_rng_scale_f16(uint64_t seed, uint64_t stream, uint64_t i);
uint16_t lb_f32_to_f16(float f);
float lb_f16_to_f32(uint16_t u);
uint16_t lb_f32_to_bf16(float f);
float lb_bf16_to_f32(uint16_t b);

#endif
