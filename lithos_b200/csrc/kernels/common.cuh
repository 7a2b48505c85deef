// Shared device helpers: mbarrier + bulk-copy (TMA) wrappers with bounded
// waits, programmatic-dependent-launch hooks, number-format helpers.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

// Device status word values written when a bounded wait gives up.  The host
// reads the word after synchronising; the kernel returns instead of trapping.
#define LB_DEV_OK 0u
#define LB_DEV_TIMEOUT_FULL 0x1001u    // consumer gave up waiting for a bulk copy
#define LB_DEV_TIMEOUT_EMPTY 0x1002u   // producer gave up waiting for a free stage
#define LB_DEV_TIMEOUT_PEER 0x1003u    // gave up waiting for a peer GPU's flag
#define LB_DEV_TIMEOUT_COUNTER 0x1004u // gave up waiting on a split counter
#define LB_DEV_POS_RANGE 0x1005u       // the decode position lies outside the KV cache: nothing was read or written

#define LB_WAIT_SPINS (1u << 22)
#define LB_WAIT_NS 2000000000ull // 2 s wall-clock cap on any single wait

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ uint64_t globaltimer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// Time limit of a wait on another CTA or GPU.  The context's status block is u32 [64]: word 0 is the status word the
// kernels get a pointer to, words 2-3 hold the limit in nanoseconds as one u64 (0 = the built-in LB_WAIT_NS).
__device__ __forceinline__ uint64_t lb_wait_limit_ns(const uint32_t* status) {
    const uint64_t v = *reinterpret_cast<const volatile uint64_t*>(status + 2);
    return v ? v : LB_WAIT_NS;
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: returns false (and the caller records a status) when the phase
// has not completed after LB_WAIT_SPINS polls or LB_WAIT_NS nanoseconds.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
    if (mbar_try_wait(bar, parity)) return true;
    uint64_t t0 = globaltimer_ns();
    for (uint32_t it = 0; it < LB_WAIT_SPINS; ++it) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((it & 255u) == 255u && globaltimer_ns() - t0 > LB_WAIT_NS) break;
    }
    return false;
}

__device__ __forceinline__ uint64_t l2_policy_evict_first() {
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}

// 1-D bulk copy global -> shared (TMA engine, no tensor map).  dst, src and
// bytes must all be multiples of 16.
__device__ __forceinline__ void bulk_g2s(void* dst_smem, const void* src_gmem, uint32_t bytes, uint64_t* bar,
                                         uint64_t policy) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(
            smem_u32(dst_smem)),
        "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar)), "l"(policy)
        : "memory");
}

// Programmatic dependent launch: a kernel may start while its predecessor in
// the stream drains.  pdl_wait() blocks until the predecessor's memory is
// visible; pdl_launch_dependents() lets the successor start its own prologue.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ float bf16_bits_to_f32(uint16_t b) { return __uint_as_float((uint32_t)b << 16); }
__device__ __forceinline__ float sigmoidf_dev(float x) { return 1.0f / (1.0f + __expf(-x)); }
__device__ __forceinline__ float siluf_dev(float x) { return x * sigmoidf_dev(x); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Block-wide sum; red must hold >= 33 floats; every thread gets the total.
// Fixed reduction order, so the result is run-to-run identical.
__device__ __forceinline__ float block_sum(float v, float* red) {
    int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) red[w] = v;
    __syncthreads();
    if (w == 0) {
        float t = lane < nw ? red[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) red[32] = t;
    }
    __syncthreads();
    return red[32];
}
