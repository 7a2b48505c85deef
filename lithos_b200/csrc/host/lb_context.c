/* Context, driver binding, kernel-image loading and the launch helper.
 *
 * This is the C re-expression of the reference's host bring-up
 * (src/launcher.s:397-520 _start, :3708-3965 load_cubins, :662-676 cuda_error):
 * CUDA driver API only — module load, function lookup, cuLaunchKernel(Ex).
 */
#define _GNU_SOURCE
#include "lb_internal.h"
#include "../kernels/params.h"
#include <dlfcn.h>
#include <stdarg.h>

lb_driver lb_drv;

static const char* const k_kernel_names[LBK_COUNT] = {
#define X(name) #name,
    LB_KERNELS(X)
#undef X
};

LB_API const char* lb_version(void) { return "lithos_b200 0.1 (sm_100a)"; }

LB_API const char* lb_status_string(int s) {
    switch (s) {
        case LB_OK: return "ok";
        case LB_ERR_INVALID: return "invalid argument";
        case LB_ERR_NO_DRIVER: return "CUDA driver or device not available";
        case LB_ERR_CUDA: return "CUDA driver call failed";
        case LB_ERR_NO_KERNEL: return "kernel image or entry point missing";
        case LB_ERR_DEVICE_WAIT: return "device-side bounded wait gave up";
        case LB_ERR_IO: return "I/O or file-format error";
        case LB_ERR_NOMEM: return "out of memory";
        case LB_ERR_STATE: return "call not valid in the current state";
        default: return "unknown status";
    }
}

int lb_fail(lb_ctx* c, int status, const char* fmt, ...) {
    if (c) {
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(c->err, sizeof c->err, fmt, ap);
        va_end(ap);
    }
    return status;
}

int lb_cu(lb_ctx* c, CUresult r, const char* what) {
    if (r == CUDA_SUCCESS) return LB_OK;
    const char* name = NULL;
    if (lb_drv.GetErrorName) lb_drv.GetErrorName(r, &name);
    /* same information the reference prints before exit(1): "lithos: CUDA error, code=N" */
    return lb_fail(c, LB_ERR_CUDA, "CUDA error, code=%d (%s) in %s", (int)r, name ? name : "?", what);
}

int lb_driver_load(char* err, size_t errlen) {
    if (lb_drv.loaded) return LB_OK;
    void* h = dlopen("libcuda.so.1", RTLD_NOW | RTLD_GLOBAL);
    if (!h) h = dlopen("libcuda.so", RTLD_NOW | RTLD_GLOBAL);
    if (!h) {
        snprintf(err, errlen, "cannot load libcuda.so.1: %s", dlerror());
        return LB_ERR_NO_DRIVER;
    }
    typedef CUresult(CUDAAPI * getproc_t)(const char*, void**, int, cuuint64_t, CUdriverProcAddressQueryResult*);
    getproc_t getproc = (getproc_t)dlsym(h, "cuGetProcAddress_v2");
    if (!getproc) {
        snprintf(err, errlen, "libcuda has no cuGetProcAddress_v2 (driver older than CUDA 12)");
        return LB_ERR_NO_DRIVER;
    }
#define X(field, sym, args)                                                                      \
    {                                                                                            \
        void* fp = NULL;                                                                         \
        CUdriverProcAddressQueryResult q;                                                        \
        CUresult r = getproc(#sym, &fp, 12040, CU_GET_PROC_ADDRESS_DEFAULT, &q);                 \
        if (r != CUDA_SUCCESS || !fp) {                                                          \
            snprintf(err, errlen, "driver entry point %s not found (code %d)", #sym, (int)r);    \
            return LB_ERR_NO_DRIVER;                                                             \
        }                                                                                        \
        *(void**)(&lb_drv.field) = fp;                                                           \
    }
    LB_DRIVER_FUNCS(X)
#undef X
    CUresult r = lb_drv.Init(0);
    if (r != CUDA_SUCCESS) {
        snprintf(err, errlen, "cuInit failed, code=%d", (int)r);
        return LB_ERR_NO_DRIVER;
    }
    lb_drv.loaded = 1;
    return LB_OK;
}

/* directory holding this shared library (kernels/ lives beside it) */
static void self_dir(char* out, size_t n) {
    Dl_info info;
    out[0] = 0;
    if (dladdr((void*)&self_dir, &info) && info.dli_fname) {
        snprintf(out, n, "%s", info.dli_fname);
        char* slash = strrchr(out, '/');
        if (slash) *slash = 0;
        else snprintf(out, n, ".");
    }
}

static int load_cubin(lb_ctx* c, const char* dir, const char* file) {
    char path[1024];
    snprintf(path, sizeof path, "%s/%s", dir, file);
    FILE* f = fopen(path, "rb");
    if (!f) return lb_fail(c, LB_ERR_NO_KERNEL, "kernel image %s not found", path);
    fseek(f, 0, SEEK_END);
    long sz = ftell(f);
    fseek(f, 0, SEEK_SET);
    void* img = malloc((size_t)sz + 1);
    if (!img || fread(img, 1, (size_t)sz, f) != (size_t)sz) {
        fclose(f);
        free(img);
        return lb_fail(c, LB_ERR_IO, "cannot read %s", path);
    }
    fclose(f);
    if (c->n_modules >= LB_MAX_MODULES) {
        free(img);
        return lb_fail(c, LB_ERR_INVALID, "too many kernel images");
    }
    CUresult r = lb_drv.ModuleLoadData(&c->modules[c->n_modules], img);
    free(img);
    if (r != CUDA_SUCCESS) return lb_cu(c, r, path);
    c->n_modules++;
    return LB_OK;
}

static const char* const k_cubins[] = {"gemv.cubin", "chain.cubin", "batched.cubin", "batched_tc.cubin", "deltanet.cubin", "attention.cubin", "attention_mma.cubin", "small.cubin", "comm.cubin", "prefill.cubin"};

LB_API int lb_init(int device, const char* kernel_dir, lb_ctx** out) {
    if (!out) return LB_ERR_INVALID;
    *out = NULL;
    lb_ctx* c = (lb_ctx*)calloc(1, sizeof *c);
    if (!c) return LB_ERR_NOMEM;
    *out = c; /* returned even on failure so the caller can read lb_last_error */
    int st = lb_driver_load(c->err, sizeof c->err);
    if (st != LB_OK) return st;
    c->device = device;
    c->pdl = 1;
    c->chain_reserve = 32 * 1024;
    LB_CU(c, lb_drv.DeviceGet(&c->cu_dev, device));
    int major = 0, minor = 0;
    LB_CU(c, lb_drv.DeviceGetAttribute(&major, CU_DEVICE_ATTRIBUTE_COMPUTE_CAPABILITY_MAJOR, c->cu_dev));
    LB_CU(c, lb_drv.DeviceGetAttribute(&minor, CU_DEVICE_ATTRIBUTE_COMPUTE_CAPABILITY_MINOR, c->cu_dev));
    if (major != 10)
        return lb_fail(c, LB_ERR_NO_KERNEL, "device %d is sm_%d%d; this library carries sm_100a code only", device, major,
                       minor);
    LB_CU(c, lb_drv.DeviceGetAttribute(&c->sm_count, CU_DEVICE_ATTRIBUTE_MULTIPROCESSOR_COUNT, c->cu_dev));
    LB_CU(c, lb_drv.DeviceGetAttribute(&c->max_smem_optin, CU_DEVICE_ATTRIBUTE_MAX_SHARED_MEMORY_PER_BLOCK_OPTIN,
                                       c->cu_dev));
    LB_CU(c, lb_drv.DevicePrimaryCtxRetain(&c->cu_ctx, c->cu_dev));
    LB_CU(c, lb_drv.CtxSetCurrent(c->cu_ctx));
    LB_CU(c, lb_drv.StreamCreate(&c->stream, CU_STREAM_NON_BLOCKING));
    LB_CU(c, lb_drv.EventCreate(&c->ev[0], CU_EVENT_DEFAULT));
    LB_CU(c, lb_drv.EventCreate(&c->ev[1], CU_EVENT_DEFAULT));

    char dir[1024];
    if (kernel_dir && kernel_dir[0]) snprintf(dir, sizeof dir, "%s", kernel_dir);
    else {
        char sd[900];
        self_dir(sd, sizeof sd);
        snprintf(dir, sizeof dir, "%s/kernels", sd);
    }
    for (size_t i = 0; i < sizeof k_cubins / sizeof k_cubins[0]; i++) LB_TRY(load_cubin(c, dir, k_cubins[i]));
    for (int k = 0; k < LBK_COUNT; k++) {
        CUresult r = CUDA_ERROR_NOT_FOUND;
        for (int m = 0; m < c->n_modules && r != CUDA_SUCCESS; m++)
            r = lb_drv.ModuleGetFunction(&c->fn[k], c->modules[m], k_kernel_names[k]);
        if (r != CUDA_SUCCESS)
            return lb_fail(c, LB_ERR_NO_KERNEL, "entry point %s not found in any kernel image under %s",
                           k_kernel_names[k], dir);
        /* let every kernel use the full opt-in shared memory (its static part counts against the same limit) */
        int stat = 0;
        LB_CU(c, lb_drv.FuncGetAttribute(&stat, CU_FUNC_ATTRIBUTE_SHARED_SIZE_BYTES, c->fn[k]));
        c->fn_static_smem[k] = stat;
        LB_CU(c, lb_drv.FuncSetAttribute(c->fn[k], CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES,
                                         c->max_smem_optin - ((stat + 1023) & ~1023)));
    }

    LB_CU(c, lb_drv.MemAlloc(&c->gemv_partial, (size_t)LB_GEMV_MAX_SPLITS * LB_GEMV_SCRATCH_N * sizeof(float)));
    LB_CU(c, lb_drv.MemAlloc(&c->gemv_counters, 4096 * sizeof(uint32_t)));
    LB_CU(c, lb_drv.MemsetD8Async(c->gemv_counters, 0, 4096 * sizeof(uint32_t), c->stream));
    c->attn_scratch_bytes = (size_t)8 * 64 * 8 * 260 * sizeof(float) + 256;
    LB_CU(c, lb_drv.MemAlloc(&c->attn_scratch, c->attn_scratch_bytes));
    LB_CU(c, lb_drv.MemsetD8Async(c->attn_scratch, 0, c->attn_scratch_bytes, c->stream));
    LB_CU(c, lb_drv.MemAlloc(&c->chain_mail, (size_t)LB_CHAIN_MAX_OPS * LB_CHAIN_MAIL_WORDS * 8));
    LB_CU(c, lb_drv.MemsetD8Async(c->chain_mail, 0, (size_t)LB_CHAIN_MAX_OPS * LB_CHAIN_MAIL_WORDS * 8, c->stream));
    c->chain_mailbox = 1;
    LB_CU(c, lb_drv.MemAlloc(&c->dev_status, 256));
    LB_CU(c, lb_drv.MemsetD8Async(c->dev_status, 0, 256, c->stream));
    c->flush_bytes = (size_t)256 << 20;
    LB_CU(c, lb_drv.MemAlloc(&c->flush_buf, c->flush_bytes));
    LB_CU(c, lb_drv.StreamSynchronize(c->stream));
    return LB_OK;
}

void lb_ops_release(lb_ctx* c);

LB_API void lb_destroy(lb_ctx* c) {
    if (!c) return;
    if (lb_drv.loaded && c->cu_ctx) {
        lb_drv.CtxSetCurrent(c->cu_ctx);
        if (c->stream) lb_drv.StreamSynchronize(c->stream);
        lb_ops_release(c);
        if (c->gemv_partial) lb_drv.MemFree(c->gemv_partial);
        if (c->gemv_counters) lb_drv.MemFree(c->gemv_counters);
        if (c->attn_scratch) lb_drv.MemFree(c->attn_scratch);
        if (c->dev_status) lb_drv.MemFree(c->dev_status);
        if (c->chain_mail) lb_drv.MemFree(c->chain_mail);
        if (c->flush_buf) lb_drv.MemFree(c->flush_buf);
        for (int m = 0; m < c->n_modules; m++) lb_drv.ModuleUnload(c->modules[m]);
        if (c->ev[0]) lb_drv.EventDestroy(c->ev[0]);
        if (c->ev[1]) lb_drv.EventDestroy(c->ev[1]);
        if (c->stream) lb_drv.StreamDestroy(c->stream);
        lb_drv.DevicePrimaryCtxRelease(c->cu_dev);
    }
    free(c);
}

LB_API const char* lb_last_error(const lb_ctx* c) { return c ? c->err : "no context"; }
LB_API int lb_device_sm_count(const lb_ctx* c) { return c ? c->sm_count : 0; }
LB_API uint64_t lb_launch_count(const lb_ctx* c) { return c ? c->launches : 0; }
LB_API void lb_launch_count_reset(lb_ctx* c) { if (c) c->launches = 0; }
LB_API void lb_set_pdl(lb_ctx* c, int on) { if (c) c->pdl = on ? 1 : 0; }
LB_API void lb_set_chain_timeline(lb_ctx* c, uint64_t buf) { if (c) c->chain_timeline = (CUdeviceptr)buf; }
LB_API void lb_set_chain_mailbox(lb_ctx* c, int on) { if (c) c->chain_mailbox = on ? 1 : 0; }
LB_API void lb_set_chain_reserve(lb_ctx* c, int bytes) { if (c && bytes >= 0 && bytes <= 128 * 1024) c->chain_reserve = bytes; }

LB_API int lb_device_status(lb_ctx* c, uint32_t* out) {
    if (!c || !out) return LB_ERR_INVALID;
    LB_CU(c, lb_drv.CtxSetCurrent(c->cu_ctx));
    LB_CU(c, lb_drv.MemcpyDtoHAsync(out, c->dev_status, 4, c->stream));
    LB_CU(c, lb_drv.StreamSynchronize(c->stream));
    if (*out != 0) {
        uint32_t st = *out;
        lb_drv.MemsetD8Async(c->dev_status, 0, 4, c->stream);
        return lb_fail(c, LB_ERR_DEVICE_WAIT, "device status 0x%x: a bounded wait inside a kernel gave up", st);
    }
    return LB_OK;
}

LB_API int lb_reset_status(lb_ctx* c) {
    if (!c) return LB_ERR_INVALID;
    LB_CU(c, lb_drv.CtxSetCurrent(c->cu_ctx));
    LB_CU(c, lb_drv.MemsetD32Async(c->dev_status, 0, 1, c->stream));
    return LB_OK;
}

/* words 2-3 of the status block: the limit the kernels' waits on other CTAs / GPUs read (common.cuh lb_wait_limit_ns) */
LB_API int lb_set_wait_limit(lb_ctx* c, uint64_t ns) {
    if (!c) return LB_ERR_INVALID;
    LB_CU(c, lb_drv.CtxSetCurrent(c->cu_ctx));
    LB_CU(c, lb_drv.MemsetD32Async(c->dev_status + 8, (unsigned)(ns & 0xffffffffu), 1, c->stream));
    LB_CU(c, lb_drv.MemsetD32Async(c->dev_status + 12, (unsigned)(ns >> 32), 1, c->stream));
    return LB_OK;
}

/* ---- memory ----------------------------------------------------------------- */
LB_API int lb_malloc(lb_ctx* c, size_t bytes, uint64_t* out) {
    if (!c || !out || bytes == 0) return lb_fail(c, LB_ERR_INVALID, "lb_malloc: bad argument");
    LB_CU(c, lb_drv.CtxSetCurrent(c->cu_ctx));
    CUdeviceptr p = 0;
    CUresult r = lb_drv.MemAlloc(&p, bytes);
    if (r == CUDA_ERROR_OUT_OF_MEMORY) return lb_fail(c, LB_ERR_NOMEM, "device out of memory allocating %zu bytes", bytes);
    LB_CU(c, r);
    *out = (uint64_t)p;
    return LB_OK;
}
LB_API int lb_free(lb_ctx* c, uint64_t p) {
    if (!c) return LB_ERR_INVALID;
    if (!p) return LB_OK;
    lb_packed_forget(c, p);
    LB_CU(c, lb_drv.CtxSetCurrent(c->cu_ctx));
    LB_CU(c, lb_drv.MemFree((CUdeviceptr)p));
    return LB_OK;
}
LB_API int lb_malloc_host(lb_ctx* c, size_t bytes, void** out) {
    if (!c || !out || bytes == 0) return lb_fail(c, LB_ERR_INVALID, "lb_malloc_host: bad argument");
    LB_CU(c, lb_drv.CtxSetCurrent(c->cu_ctx));
    LB_CU(c, lb_drv.MemHostAlloc(out, bytes, 0));
    return LB_OK;
}
LB_API int lb_free_host(lb_ctx* c, void* p) {
    if (!c) return LB_ERR_INVALID;
    if (!p) return LB_OK;
    LB_CU(c, lb_drv.MemFreeHost(p));
    return LB_OK;
}
LB_API int lb_memcpy_h2d(lb_ctx* c, uint64_t dst, const void* src, size_t bytes) {
    if (!c || !dst || !src) return lb_fail(c, LB_ERR_INVALID, "lb_memcpy_h2d: NULL argument");
    LB_CU(c, lb_drv.MemcpyHtoDAsync((CUdeviceptr)dst, src, bytes, c->stream));
    return LB_OK;
}
LB_API int lb_memcpy_d2h(lb_ctx* c, void* dst, uint64_t src, size_t bytes) {
    if (!c || !dst || !src) return lb_fail(c, LB_ERR_INVALID, "lb_memcpy_d2h: NULL argument");
    LB_CU(c, lb_drv.MemcpyDtoHAsync(dst, (CUdeviceptr)src, bytes, c->stream));
    return LB_OK;
}
LB_API int lb_memcpy_d2d(lb_ctx* c, uint64_t dst, uint64_t src, size_t bytes) {
    if (!c || !dst || !src) return lb_fail(c, LB_ERR_INVALID, "lb_memcpy_d2d: NULL argument");
    LB_CU(c, lb_drv.MemcpyDtoDAsync((CUdeviceptr)dst, (CUdeviceptr)src, bytes, c->stream));
    return LB_OK;
}
LB_API int lb_memset(lb_ctx* c, uint64_t dst, int v, size_t bytes) {
    if (!c || !dst) return lb_fail(c, LB_ERR_INVALID, "lb_memset: NULL argument");
    LB_CU(c, lb_drv.MemsetD8Async((CUdeviceptr)dst, (unsigned char)v, bytes, c->stream));
    return LB_OK;
}
LB_API int lb_sync(lb_ctx* c) {
    if (!c) return LB_ERR_INVALID;
    LB_CU(c, lb_drv.StreamSynchronize(c->stream));
    return LB_OK;
}

/* ---- timing -------------------------------------------------------------------- */
LB_API int lb_timer_start(lb_ctx* c) {
    if (!c) return LB_ERR_INVALID;
    LB_CU(c, lb_drv.EventRecord(c->ev[0], c->stream));
    return LB_OK;
}
LB_API int lb_timer_stop(lb_ctx* c, float* ms) {
    if (!c || !ms) return LB_ERR_INVALID;
    LB_CU(c, lb_drv.EventRecord(c->ev[1], c->stream));
    LB_CU(c, lb_drv.EventSynchronize(c->ev[1]));
    LB_CU(c, lb_drv.EventElapsedTime(ms, c->ev[0], c->ev[1]));
    return LB_OK;
}
LB_API int lb_flush_l2(lb_ctx* c) {
    if (!c) return LB_ERR_INVALID;
    static uint32_t tag = 1;
    size_t n16 = c->flush_bytes / 16;
    uint32_t t = tag++;
    void* params[] = {&c->flush_buf, &n16, &t};
    return lb_launch(c, LBK_l2_flush, (unsigned)c->sm_count * 8, 1, 1, 256, 0, params, 0);
}

/* ---- launch: replaces the cuLaunchKernel call sites (src/launcher.s:744-762) ---- */
int lb_launch(lb_ctx* c, int kernel, unsigned gx, unsigned gy, unsigned gz, unsigned bx, unsigned smem, void** params,
              int pdl) {
    return lb_launch_cluster(c, kernel, gx, gy, gz, bx, smem, params, pdl, 1);
}

/* cluster_y > 1: the gy CTAs of a column are launched as one thread-block cluster (gy % cluster_y == 0) */
int lb_launch_cluster(lb_ctx* c, int kernel, unsigned gx, unsigned gy, unsigned gz, unsigned bx, unsigned smem,
                      void** params, int pdl, unsigned cluster_y) {
    if (!c->fn[kernel]) return lb_fail(c, LB_ERR_NO_KERNEL, "kernel %s not loaded", k_kernel_names[kernel]);
    if (gx == 0 || gy == 0 || gz == 0) return lb_fail(c, LB_ERR_INVALID, "empty grid for %s", k_kernel_names[kernel]);
    if ((int)smem > c->max_smem_optin - ((c->fn_static_smem[kernel] + 1023) & ~1023))
        return lb_fail(c, LB_ERR_INVALID, "%s needs %u B of dynamic shared memory (> %d)", k_kernel_names[kernel], smem,
                       c->max_smem_optin - ((c->fn_static_smem[kernel] + 1023) & ~1023));
    CUlaunchConfig cfg;
    memset(&cfg, 0, sizeof cfg);
    cfg.gridDimX = gx; cfg.gridDimY = gy; cfg.gridDimZ = gz;
    cfg.blockDimX = bx; cfg.blockDimY = 1; cfg.blockDimZ = 1;
    cfg.sharedMemBytes = smem;
    cfg.hStream = c->stream;
    CUlaunchAttribute attr[2];
    memset(attr, 0, sizeof attr);
    unsigned na = 0;
    if (pdl && c->pdl) {
        attr[na].id = CU_LAUNCH_ATTRIBUTE_PROGRAMMATIC_STREAM_SERIALIZATION;
        attr[na].value.programmaticStreamSerializationAllowed = 1;
        na++;
    }
    if (cluster_y > 1) {
        if (gy % cluster_y) return lb_fail(c, LB_ERR_INVALID, "grid.y %u not a multiple of the cluster size %u", gy, cluster_y);
        attr[na].id = CU_LAUNCH_ATTRIBUTE_CLUSTER_DIMENSION;
        attr[na].value.clusterDim.x = 1;
        attr[na].value.clusterDim.y = cluster_y;
        attr[na].value.clusterDim.z = 1;
        na++;
    }
    if (na) {
        cfg.attrs = attr;
        cfg.numAttrs = na;
    }
    CUresult r = lb_drv.LaunchKernelEx(&cfg, c->fn[kernel], params, NULL);
    if (r != CUDA_SUCCESS) return lb_cu(c, r, k_kernel_names[kernel]);
    c->launches++;
    return LB_OK;
}

/* ---- generic module load + launch --------------------------------------------
 * The exact mechanism the reference launcher uses for every kernel:
 * load_one_cubin = read file + cuModuleLoadData + cuModuleGetFunction
 * (src/launcher.s:3861-3965) and cuLaunchKernel with a void** parameter array
 * (src/launcher.s:744-762).  Lets a caller drive any cubin that keeps the
 * reference's entry names and parameter blocks through this library. */
LB_API int lb_module_load(lb_ctx* c, const char* cubin_path, int* module_out) {
    if (!c || !cubin_path || !module_out) return lb_fail(c, LB_ERR_INVALID, "lb_module_load: NULL argument");
    LB_CU(c, lb_drv.CtxSetCurrent(c->cu_ctx));
    const char* slash = strrchr(cubin_path, '/');
    char dir[1024];
    if (slash) {
        size_t n = (size_t)(slash - cubin_path);
        if (n >= sizeof dir) return lb_fail(c, LB_ERR_INVALID, "lb_module_load: path too long");
        memcpy(dir, cubin_path, n);
        dir[n] = 0;
    } else snprintf(dir, sizeof dir, ".");
    LB_TRY(load_cubin(c, dir, slash ? slash + 1 : cubin_path));
    *module_out = c->n_modules - 1;
    return LB_OK;
}

LB_API int lb_module_get_kernel(lb_ctx* c, int module, const char* entry, uint64_t* kernel_out) {
    if (!c || !entry || !kernel_out || module < 0 || module >= c->n_modules)
        return lb_fail(c, LB_ERR_INVALID, "lb_module_get_kernel: bad argument");
    CUfunction f = NULL;
    CUresult r = lb_drv.ModuleGetFunction(&f, c->modules[module], entry);
    if (r != CUDA_SUCCESS) return lb_fail(c, LB_ERR_NO_KERNEL, "entry point %s not found in module %d", entry, module);
    lb_drv.FuncSetAttribute(f, CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES, c->max_smem_optin - 1024);
    *kernel_out = (uint64_t)(uintptr_t)f;
    return LB_OK;
}

LB_API int lb_launch_kernel(lb_ctx* c, uint64_t kernel, unsigned gx, unsigned gy, unsigned gz, unsigned bx, unsigned by,
                            unsigned bz, unsigned smem_bytes, void** params) {
    if (!c || !kernel || !params) return lb_fail(c, LB_ERR_INVALID, "lb_launch_kernel: NULL argument");
    if (!gx || !gy || !gz || !bx || !by || !bz) return lb_fail(c, LB_ERR_INVALID, "lb_launch_kernel: empty grid or block");
    LB_CU(c, lb_drv.LaunchKernel((CUfunction)(uintptr_t)kernel, gx, gy, gz, bx, by, bz, smem_bytes, c->stream, params, NULL));
    c->launches++;
    return LB_OK;
}

/* ---- CUDA graphs -----------------------------------------------------------------
 * The reference submits ~1000 launches per token one by one and synchronises after each
 * (debug_sync_tag, src/launcher.s:4044-4096); its design notes aim at one submission per
 * token (src/launcher.ls:16-106).  Here any sequence of this library's launches on the
 * context stream can be captured once and replayed as a single graph launch;
 * programmatic-dependent-launch edges between consecutive kernels are kept. */
struct lb_graph {
    CUgraph graph;
    CUgraphExec exec;
    size_t kernel_nodes;
};

LB_API int lb_graph_begin_capture(lb_ctx* c) {
    if (!c) return LB_ERR_INVALID;
    if (c->capturing) return lb_fail(c, LB_ERR_STATE, "capture already in progress");
    LB_CU(c, lb_drv.CtxSetCurrent(c->cu_ctx));
    LB_CU(c, lb_drv.StreamBeginCapture(c->stream, CU_STREAM_CAPTURE_MODE_THREAD_LOCAL));
    c->capturing = 1;
    c->capture_launches0 = c->launches;
    return LB_OK;
}

LB_API int lb_graph_end_capture(lb_ctx* c, lb_graph** out) {
    if (!c || !out) return LB_ERR_INVALID;
    if (!c->capturing) return lb_fail(c, LB_ERR_STATE, "no capture in progress");
    c->capturing = 0;
    lb_graph* g = (lb_graph*)calloc(1, sizeof *g);
    if (!g) return LB_ERR_NOMEM;
    CUresult r = lb_drv.StreamEndCapture(c->stream, &g->graph);
    if (r != CUDA_SUCCESS) { free(g); return lb_cu(c, r, "cuStreamEndCapture"); }
    g->kernel_nodes = (size_t)(c->launches - c->capture_launches0);
    c->launches = c->capture_launches0; /* captured launches have not run */
    r = lb_drv.GraphInstantiate(&g->exec, g->graph, 0);
    if (r != CUDA_SUCCESS) { lb_drv.GraphDestroy(g->graph); free(g); return lb_cu(c, r, "cuGraphInstantiate"); }
    *out = g;
    return LB_OK;
}

LB_API int lb_graph_launch(lb_ctx* c, lb_graph* g) {
    if (!c || !g) return LB_ERR_INVALID;
    if (c->capturing) return lb_fail(c, LB_ERR_STATE, "graph launch during capture");
    LB_CU(c, lb_drv.GraphLaunch(g->exec, c->stream));
    c->launches += g->kernel_nodes;
    return LB_OK;
}

LB_API int lb_graph_kernel_count(const lb_graph* g) { return g ? (int)g->kernel_nodes : 0; }

LB_API void lb_graph_destroy(lb_ctx* c, lb_graph* g) {
    if (!g) return;
    if (lb_drv.loaded) {
        if (g->exec) lb_drv.GraphExecDestroy(g->exec);
        if (g->graph) lb_drv.GraphDestroy(g->graph);
    }
    free(g);
}
