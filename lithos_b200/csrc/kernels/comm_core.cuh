// The rendezvous of the tensor-parallel exchange, shared by the stand-alone kernels (comm.cu) and the all-reduce
// entries of the persistent decode chain (chain.cu).  One thread block per GPU runs it.
#pragma once
#include "common.cuh"
#include "params.h"

__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// 8-byte accesses that are not cached in L1 and are delivered whole: the (value, generation) words of the pushed exchange
__device__ __forceinline__ void st_volatile_u64(unsigned long long* p, unsigned long long v) {
    asm volatile("st.volatile.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_volatile_u64(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.volatile.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}

// two neighbouring 8-byte words in one 16-byte load (each word was stored whole, so each is seen whole)
__device__ __forceinline__ uint4 ld_volatile_v4(const unsigned long long* p) {
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}

// returns false when a peer did not show up in time
__device__ __forceinline__ bool tp_rendezvous(const lb_tp_params& p, unsigned g, bool* s_ok) {
    const int t = threadIdx.x;
    if (t == 0) *s_ok = true;
    __syncthreads();
    if (t < p.size) {
        __threadfence_system(); // the partial written by the previous kernel is visible to peers before the flag
        st_release_sys(p.peer_flags[t] + p.rank, g);
        const uint64_t t0 = globaltimer_ns(), limit = lb_wait_limit_ns(p.status);
        bool ok = false;
        // a wait that already ran out in this context is not repeated: every later exchange returns at once,
        // so a lost peer costs one time limit, not one per exchange
        const bool dead = *reinterpret_cast<volatile unsigned*>(p.status) != 0u;
        for (unsigned it = 0; it < LB_WAIT_SPINS && !dead; ++it) {
            // generations only grow; (int) difference keeps the test valid across wrap-around
            if ((int)(ld_acquire_sys(p.my_flags + t) - g) >= 0) { ok = true; break; }
            if ((it & 63u) == 63u && globaltimer_ns() - t0 > limit) break;
        }
        if (!ok) { atomicCAS(p.status, 0u, LB_DEV_TIMEOUT_PEER); *s_ok = false; }
    }
    __syncthreads();
    return *s_ok;
}

