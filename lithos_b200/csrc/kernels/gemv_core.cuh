// Pieces shared by the int4 GEMV kernels (one GEMV per launch in gemv.cu, a chain of GEMVs per
// launch in chain.cu): the tiled TMA loads of a weight stage, the integer tensor-core step, the
// digit-table layout and the activation prologue.
#pragma once
#include "common.cuh"
#include "params.h"

#define GEMV_BOX_BYTES (LB_GEMV_ROWS * 128)  // one swizzled box: 16 packed rows x 32 columns
#define GEMV_STAGE_BYTES LB_GEMV_STAGE_BYTES // eight boxes side by side = one group x 256 columns

// One tiled TMA load (no multicast) of a whole stage: the tensor map views qweight as
// [column block of 32][packed row][32 columns]; the box is 8 column blocks x 16 rows x 32
// columns, written as eight consecutive 2 KB boxes with the 128-byte swizzle.
__device__ __forceinline__ void tma_load_stage(uint32_t dst_smem, const void* tmap, int colblock, int row, uint64_t* bar,
                                               uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint"
        " [%0], [%1, {%2, %3, %4}], [%5], %6;" ::"r"(dst_smem),
        "l"(tmap), "r"(0), "r"(row), "r"(colblock), "r"(smem_u32(bar)), "l"(policy)
        : "memory");
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst_smem, const void* tmap, int x, int y, uint64_t* bar, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint"
        " [%0], [%1, {%2, %3}], [%4], %5;" ::"r"(dst_smem),
        "l"(tmap), "r"(x), "r"(y), "r"(smem_u32(bar)), "l"(policy)
        : "memory");
}

// D(16x8, s32) += A(16x32, u8) * B(32x8, s8)
__device__ __forceinline__ void imma16832(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                          uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Two packed words of one packed row (column cA -> fragment row g, cB -> row g+8) against the
// activation digits of that row.  w & 0x0f0f0f0f are the even nibbles (k = 0,2,4,6) as four
// u8, (w >> 4) & 0x0f0f0f0f the odd ones: the whole int4 -> operand conversion is 3
// instructions per 8 weights, and the products are exact integers.
__device__ __forceinline__ void imma_words(int (&d)[4], uint32_t cA, uint32_t cB, uint2 xb) {
    const uint32_t M = 0x0f0f0f0fu;
    imma16832(d, cA & M, cB & M, (cA >> 4) & M, (cB >> 4) & M, xb.x, xb.y);
}

// word offset of packed row R in the digit table: 6 words (3 planes x 8 bytes) per row plus a
// 2-word pad every 4 rows, which makes the per-step fragment loads bank-conflict free
__device__ __forceinline__ int digit_row_word(int R) { return 6 * R + 2 * (R >> 2); }

// The activation of one packed row (8 consecutive k) as the kernel uses it: fp32 values already
// rounded to fp16 (the activation contract), after the optional norm prologue.
// P is any parameter block with x, aux0, aux1, x_mode and eps.  CG = true reads x and the gate through
// L2 only (ld.global.cg): required when another CTA of the SAME launch produced them.
template <bool CG, class P>
__device__ __forceinline__ void load_x_row(const P& p, int k, bool live, float rinv, float (&v)[8]) {
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = 0.f;
    if (live) {
        if (p.x_mode == LB_X_F16) {
            const uint4* xp = reinterpret_cast<const uint4*>(reinterpret_cast<const __half*>(p.x) + k);
            uint4 raw = CG ? __ldcg(xp) : __ldg(xp);
            const __half2* h = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                float2 f = __half22float2(h[j]);
                v[2 * j] = f.x;
                v[2 * j + 1] = f.y;
            }
        } else {
            const float4* xv = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p.x) + k);
            float4 a = CG ? __ldcg(xv) : __ldg(xv), b = CG ? __ldcg(xv + 1) : __ldg(xv + 1);
            v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
            v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
        }
    }
    if (p.x_mode == LB_X_F32_RMSNORM) {
        if (live) {
            uint4 wr = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(p.aux0) + k));
            const uint16_t* wb = reinterpret_cast<const uint16_t*>(&wr);
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = v[j] * rinv * (1.0f + bf16_bits_to_f32(wb[j]));
        }
    } else if (p.x_mode == LB_X_F32_HEADNORM_SILU) {
        // one head = 128 values = the 16 rows held by a 16-lane segment (called by full warps)
        float ss = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) ss += v[j] * v[j];
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        float hr = rsqrtf(ss * (1.0f / 128.0f) + p.eps);
        if (live) {
            const float4* zv = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p.aux1) + k);
            const float4* wv = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p.aux0) + (k & 127));
            float4 za = CG ? __ldcg(zv) : __ldg(zv), zb = CG ? __ldcg(zv + 1) : __ldg(zv + 1), wa = __ldg(wv), wb = __ldg(wv + 1);
            float z[8] = {za.x, za.y, za.z, za.w, zb.x, zb.y, zb.z, zb.w};
            float w[8] = {wa.x, wa.y, wa.z, wa.w, wb.x, wb.y, wb.z, wb.w};
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = v[j] * hr * w[j] * siluf_dev(z[j]);
        }
    }
    if (p.x_mode != LB_X_F16) {
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = __half2float(__float2half_rn(v[j]));
    }
}

