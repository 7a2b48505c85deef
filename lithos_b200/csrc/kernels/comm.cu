// Tensor-parallel exchange kernels over NVLink peer memory (one process per GPU).
//
// The reference is single-GPU; these have no counterpart there.  A row-parallel
// projection leaves this GPU's partial [hidden] vector in its own exchange buffer
// (mapped into every peer through CUDA IPC).  tp_allreduce_add then
//   1. publishes "my partial of generation g is complete" by writing g into slot
//      [my_rank] of every peer's flag array (system-scope release),
//   2. waits until its own flag array shows generation g for every rank (bounded
//      spin: on expiry a status word is set and the kernel returns, no trap),
//   3. reads all partials with plain loads, adds them in RANK ORDER (every GPU gets
//      bit-identical sums) and adds the result to the residual stream.
// Partials are double-buffered by call parity: a GPU can only reach generation g+2
// after every peer has published g+1, i.e. after every peer has finished reading g.
// No multicast, no TMA on peer memory: plain ld/st only.
#include "comm_core.cuh"

extern "C" __global__ void __launch_bounds__(1024) tp_allreduce_add(const __grid_constant__ lb_tp_params p) {
    __shared__ bool s_ok;
    pdl_wait();
    const unsigned g = p.gen[0] + 1u;
    const bool ok = tp_rendezvous(p, g, &s_ok);
    pdl_launch_dependents();
    if (ok) {
        for (int i = threadIdx.x; i < p.n; i += blockDim.x) {
            float s = 0.f;
            for (int r = 0; r < p.size; ++r) s += __ldcv(p.partials[r] + LB_TP_PARTIAL(p, p.slot, r) + i); // rank order
            p.x[i] += s;
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) p.gen[0] = g;
}

// Greedy sampling across vocabulary shards: every rank contributes its best (logit, token) and
// every rank picks the same winner (greater logit, smaller token on ties).
extern "C" __global__ void __launch_bounds__(1024) tp_argmax_exchange(const __grid_constant__ lb_tp_argmax_params q) {
    __shared__ float sv[32];
    __shared__ int si[32];
    __shared__ bool s_ok;
    const lb_tp_params& p = q.tp;
    pdl_wait();
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < q.n_cand; i += blockDim.x) {
        const float v = q.cand_val[i];
        const int id = q.cand_idx[i];
        if (v > bv || (v == bv && id < bi)) { bv = v; bi = id; }
    }
    auto better = [](float v, int i, float bv2, int bi2) { return v > bv2 || (v == bv2 && i < bi2); };
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
    }
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    if (lane == 0) { sv[w] = bv; si[w] = bi; }
    __syncthreads();
    if (w == 0) {
        const int nw = blockDim.x >> 5;
        bv = lane < nw ? sv[lane] : -INFINITY;
        bi = lane < nw ? si[lane] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
        }
        if (lane == 0) { // publish (logit, global token) in this rank's exchange buffer
            float* mine = p.partials[p.rank] + LB_TP_PARTIAL(p, 2, 0) + 2 * p.rank; // every rank its own pair of words
            mine[0] = bv;
            reinterpret_cast<int*>(mine)[1] = bi == 0x7fffffff ? 0x7fffffff : bi + q.vocab_offset;
        }
    }
    __syncthreads();
    const unsigned g = p.gen[0] + 1u;
    const bool ok = tp_rendezvous(p, g, &s_ok);
    if (threadIdx.x == 0) {
        float gv = -INFINITY;
        int gi = 0x7fffffff;
        if (ok)
            for (int r = 0; r < p.size; ++r) {
                const float* rec = p.partials[r] + LB_TP_PARTIAL(p, 2, 0) + 2 * r;
                const float v = __ldcv(rec);
                const int id = __ldcv(reinterpret_cast<const int*>(rec) + 1);
                if (better(v, id, gv, gi)) { gv = v; gi = id; }
            }
        if (gi == 0x7fffffff) gi = 0;
        q.out_idx[0] = gi;
        if (q.next_token) q.next_token[0] = gi;
        if (q.pos) q.pos[0] += 1;
        p.gen[0] = g;
    }
}
