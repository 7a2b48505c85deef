// lb_attention_decode_noalloc: the GQA decode-attention call for callers that must not allocate.
//
// Who needs it: code that runs where device allocation is off the table — a step that is being
// recorded into a CUDA graph by the caller, a real-time loop that pre-sized everything at start-up,
// a plugin living inside another runtime's memory pool, a process that shares the GPU and was
// given a fixed memory budget.  lb_attention_decode takes its split-KV scratch from the context
// (allocated in lb_init); this entry point needs no context at all: the scratch is a fixed array
// inside this library's device image, so loading the library is the only "allocation" there is
// (every GPU that loads it holds NOALLOC_SCRATCH_BYTES until the process exits).
//
// It launches attn_decode_split (included below: CUDA-core dot products, split-KV with a last-arriver merge) with at
// most NOALLOC_MAX_SLICES position slices per KV head; lb_attention_decode itself uses the tensor-core kernel
// attn_decode_mma.  Same contract and results to rounding; tests/test_zz_no_alloc.py checks both against the CPU oracle.
//
// Threads: the per-device address cache below is filled by the first call on a device without a lock.  Two host
// threads making that first call at the same moment would both store the same address (harmless), but make the
// first call from one thread.
#include <cuda_runtime.h>
#include <cstdio>
#include <cstring>
#include <cmath>

#include "../kernels/attention.cu"
#include "lithos_b200.h"

#define NOALLOC_MAX_KV_HEADS 8
#define NOALLOC_MAX_SLICES 16
#define NOALLOC_MAX_GROUP 6
#define NOALLOC_RECORD_FLOATS ((size_t)NOALLOC_MAX_KV_HEADS * NOALLOC_MAX_SLICES * NOALLOC_MAX_GROUP * AT_REC)
#define NOALLOC_COUNTER_WORDS 64
#define NOALLOC_SCRATCH_BYTES (NOALLOC_RECORD_FLOATS * 4 + NOALLOC_COUNTER_WORDS * 4) /* 798 976 bytes */
#define NOALLOC_MAX_DEVICES 64

// Slice records [kv][slice][head][260] followed by one arrival counter per KV head.  In host code
// this name is only a stand-in for the symbol, not an address a kernel could use: the device
// address is looked up once per device with cudaGetSymbolAddress.
static __device__ __align__(256) float g_noalloc_scratch[NOALLOC_SCRATCH_BYTES / 4];

static float* g_scratch_addr[NOALLOC_MAX_DEVICES]; // per device, resolved on the first call there

static int fail(char* err, size_t errlen, int status, const char* what, cudaError_t e) {
    if (err && errlen) {
        if (e != cudaSuccess) snprintf(err, errlen, "%s: %s", what, cudaGetErrorString(e));
        else snprintf(err, errlen, "%s", what);
    }
    return status;
}

extern "C" __attribute__((visibility("default"))) int lb_attention_decode_noalloc(
    void* stream, uint64_t q, uint64_t k_new, uint64_t v_new, uint64_t gate, uint64_t q_norm_w, uint64_t k_norm_w,
    uint64_t k_cache, uint64_t v_cache, uint64_t out, int pos, int HQ, int HKV, int in_is_f32, int rot_dims,
    float rope_theta, float eps, char* err, size_t errlen) {
    if (!q || !k_new || !v_new || !k_cache || !v_cache || !out || pos < 0 || HKV <= 0 || HQ <= 0 || HQ % HKV)
        return fail(err, errlen, LB_ERR_INVALID, "lb_attention_decode_noalloc: bad argument", cudaSuccess);
    const int G = HQ / HKV;
    if (HKV > NOALLOC_MAX_KV_HEADS || G > NOALLOC_MAX_GROUP || !(G == 1 || G == 2 || G == 3 || G == 4 || G == 6))
        return fail(err, errlen, LB_ERR_INVALID,
                    "lb_attention_decode_noalloc: at most 8 KV heads and 1, 2, 3, 4 or 6 query heads per KV head fit the built-in scratch",
                    cudaSuccess);
    if ((q_norm_w == 0) != (k_norm_w == 0) || rot_dims < 0 || rot_dims > 128 || rot_dims % 8)
        return fail(err, errlen, LB_ERR_INVALID, "lb_attention_decode_noalloc: bad norm weights or rot_dims", cudaSuccess);

    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return fail(err, errlen, LB_ERR_NO_DRIVER, "cudaGetDevice", e);
    if (dev < 0 || dev >= NOALLOC_MAX_DEVICES) return fail(err, errlen, LB_ERR_INVALID, "device index out of range", cudaSuccess);
    if (!g_scratch_addr[dev]) {
        // first call on this device (it is the current one): resolve the array's device address and
        // let the kernel use its dynamic shared memory.  Neither call allocates.
        float* p = nullptr;
        e = cudaGetSymbolAddress((void**)&p, g_noalloc_scratch);
        if (e != cudaSuccess || !p) return fail(err, errlen, LB_ERR_CUDA, "cudaGetSymbolAddress(scratch)", e);
        e = cudaFuncSetAttribute(attn_decode_split, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024);
        if (e != cudaSuccess) return fail(err, errlen, LB_ERR_CUDA, "cudaFuncSetAttribute", e);
        g_scratch_addr[dev] = p;
    }
    float* scratch = g_scratch_addr[dev];

    lb_attn_params p;
    memset(&p, 0, sizeof p);
    p.q = (const void*)q; p.k_new = (const void*)k_new; p.v_new = (const void*)v_new; p.gate = (const void*)gate;
    p.q_norm_w = (const uint16_t*)q_norm_w; p.k_norm_w = (const uint16_t*)k_norm_w;
    p.k_cache = (uint16_t*)k_cache; p.v_cache = (uint16_t*)v_cache; p.out = (float*)out;
    p.scratch = scratch;
    p.counters = reinterpret_cast<uint32_t*>(scratch + NOALLOC_RECORD_FLOATS);
    p.pos = pos; p.HQ = HQ; p.HKV = HKV;
    int splits = pos / 64;
    if (splits < 1) splits = 1;
    if (splits > NOALLOC_MAX_SLICES) splits = NOALLOC_MAX_SLICES;
    p.splits = splits;
    p.in_dtype = in_is_f32 ? 1 : 0;
    p.gate_stride = 256; p.q_stride = 256;
    p.rot_dims = rot_dims; p.rope_theta = rope_theta; p.eps = eps;
    for (int i = 0; i < rot_dims / 2; i++) p.rope_freq[i] = exp2(-log2((double)rope_theta) * (double)i / (double)(rot_dims / 2));

    cudaStream_t st = (cudaStream_t)stream;
    // the array keeps whatever the last call left: the arrival counters must start at zero
    e = cudaMemsetAsync(p.counters, 0, NOALLOC_COUNTER_WORDS * 4, st);
    if (e != cudaSuccess) return fail(err, errlen, LB_ERR_CUDA, "cudaMemsetAsync(counters)", e);
    const unsigned smem = (unsigned)((G * 256 + 256 + 256 + 40 + 2 * 8 * 8 + 8 * G * 256) * 4 + 64);
    attn_decode_split<<<dim3((unsigned)HKV, (unsigned)splits, 1), 256, smem, st>>>(p);
    e = cudaGetLastError();
    if (e != cudaSuccess) return fail(err, errlen, LB_ERR_CUDA, "launch of attn_decode_split", e);
    return LB_OK;
}
