/* Tensor-parallel exchange buffers: one process per GPU, peers mapped through CUDA IPC.
 * No counterpart in the reference (single GPU, no collective anywhere). */
#include "lb_internal.h"
#include "../kernels/params.h"

struct lb_comm {
    lb_ctx* c;
    int rank, size, n_max;
    size_t flags_off, words_off, bytes;
    CUdeviceptr buf;              /* this rank's buffer: float [2][size][n_max] partials | float [n_max] sampling record |
                                     unsigned flags [8] | unsigned gen | u64 [2][size][n_max] (value, generation) words (params.h) */
    CUdeviceptr peer[LB_TP_MAX];  /* every rank's buffer as seen from this GPU (peer[rank] == buf) */
    int opened[LB_TP_MAX];
};

LB_API int lb_comm_create(lb_ctx* c, int rank, int size, int n_max, lb_comm** out) {
    if (!c || !out || size < 1 || size > LB_TP_MAX || rank < 0 || rank >= size || n_max < 16)
        return lb_fail(c, LB_ERR_INVALID, "lb_comm_create: bad argument");
    lb_comm* m = (lb_comm*)calloc(1, sizeof *m);
    if (!m) return LB_ERR_NOMEM;
    m->c = c; m->rank = rank; m->size = size; m->n_max = n_max;
    m->flags_off = ((size_t)(2 * size + 1) * n_max * 4 + 255) & ~(size_t)255;
    m->words_off = m->flags_off + 256;
    m->bytes = m->words_off + (size_t)2 * size * n_max * 8;
    LB_CU(c, lb_drv.CtxSetCurrent(c->cu_ctx));
    CUresult r = lb_drv.MemAlloc(&m->buf, m->bytes);
    if (r != CUDA_SUCCESS) { free(m); return lb_cu(c, r, "cuMemAlloc(exchange buffer)"); }
    lb_drv.MemsetD8Async(m->buf, 0, m->bytes, c->stream);
    lb_drv.StreamSynchronize(c->stream);
    m->peer[rank] = m->buf;
    *out = m;
    return LB_OK;
}

LB_API int lb_comm_rank(const lb_comm* m) { return m ? m->rank : -1; }
LB_API int lb_comm_size(const lb_comm* m) { return m ? m->size : 0; }

/* 64-byte IPC handle of this rank's buffer, to be sent to every peer by the launcher */
LB_API int lb_comm_handle(lb_comm* m, void* handle_out64) {
    if (!m || !handle_out64) return LB_ERR_INVALID;
    CUipcMemHandle h;
    LB_CU(m->c, lb_drv.IpcGetMemHandle(&h, m->buf));
    memcpy(handle_out64, &h, sizeof h);
    return LB_OK;
}

/* handles: size x 64 bytes, in rank order (this rank's own entry is ignored) */
LB_API int lb_comm_open(lb_comm* m, const void* handles) {
    if (!m || !handles) return LB_ERR_INVALID;
    LB_CU(m->c, lb_drv.CtxSetCurrent(m->c->cu_ctx));
    for (int r = 0; r < m->size; r++) {
        if (r == m->rank || m->opened[r]) continue;
        CUipcMemHandle h;
        memcpy(&h, (const unsigned char*)handles + (size_t)r * sizeof h, sizeof h);
        LB_CU(m->c, lb_drv.IpcOpenMemHandle(&m->peer[r], h, CU_IPC_MEM_LAZY_ENABLE_PEER_ACCESS));
        m->opened[r] = 1;
    }
    return LB_OK;
}

/* a peer's buffer that this process can already address: another GPU of the same process with peer access enabled, or
 * (tests) a local stand-in for a rank that never answers */
LB_API int lb_comm_set_peer(lb_comm* m, int rank, uint64_t peer_buffer) {
    if (!m || rank < 0 || rank >= m->size || rank == m->rank || !peer_buffer || (peer_buffer & 255))
        return lb_fail(m ? m->c : NULL, LB_ERR_INVALID, "lb_comm_set_peer: bad rank or buffer (256-byte aligned, lb_comm_bytes long)");
    if (m->opened[rank]) return lb_fail(m->c, LB_ERR_STATE, "lb_comm_set_peer: rank %d is already opened through its IPC handle", rank);
    m->peer[rank] = (CUdeviceptr)peer_buffer;
    return LB_OK;
}
LB_API size_t lb_comm_bytes(const lb_comm* m) { return m ? m->bytes : 0; }
LB_API uint64_t lb_comm_buffer(const lb_comm* m) { return m ? (uint64_t)m->buf : 0; }
LB_API size_t lb_comm_flags_offset(const lb_comm* m) { return m ? m->flags_off : 0; }

LB_API void lb_comm_destroy(lb_comm* m) {
    if (!m) return;
    if (lb_drv.loaded && m->c && m->c->cu_ctx) {
        lb_drv.CtxSetCurrent(m->c->cu_ctx);
        lb_drv.StreamSynchronize(m->c->stream);
        for (int r = 0; r < m->size; r++)
            if (m->opened[r]) lb_drv.IpcCloseMemHandle(m->peer[r]);
        if (m->buf) lb_drv.MemFree(m->buf);
    }
    free(m);
}

/* fill the device-side description used by the exchange kernels */
int lb_comm_fill(const lb_comm* m, lb_tp_params* p, int slot, int n) {
    memset(p, 0, sizeof *p);
    for (int r = 0; r < m->size; r++) {
        if (!m->peer[r]) return lb_fail(m->c, LB_ERR_STATE, "exchange buffer of rank %d not opened", r);
        p->partials[r] = (float*)m->peer[r];
        p->peer_flags[r] = (unsigned*)(m->peer[r] + m->flags_off);
        p->words[r] = (unsigned long long*)(m->peer[r] + m->words_off);
    }
    p->my_flags = (unsigned*)(m->buf + m->flags_off);
    p->gen = (unsigned*)(m->buf + m->flags_off + 128);
    p->status = (unsigned*)m->c->dev_status;
    p->n = n; p->n_max = m->n_max; p->slot = slot; p->rank = m->rank; p->size = m->size;
    return LB_OK;
}

/* one exchange outside the decode step: x[0..n) += sum over ranks of their partial vectors in `slot` (0 or 1; every rank
 * has written its own partial to lb_comm_buffer + slot * n_max * 4 before the call) */
LB_API int lb_comm_allreduce(lb_comm* m, uint64_t x, int n, int slot) {
    if (!m || !x || n < 1 || n > m->n_max || slot < 0 || slot > 1) return lb_fail(m ? m->c : NULL, LB_ERR_INVALID, "lb_comm_allreduce: bad argument");
    lb_tp_params p;
    LB_TRY(lb_comm_fill(m, &p, slot, n));
    p.x = (float*)x;
    void* params[] = {&p};
    return lb_launch(m->c, LBK_tp_allreduce_add, 1, 1, 1, 1024, 0, params, 1);
}

/* where rank `rank`'s partial vector of exchange slot `slot` lives inside an exchange buffer (bytes from its start) */
LB_API size_t lb_comm_partial_offset(const lb_comm* m, int slot, int rank) {
    if (!m) return 0;
    return (size_t)(slot == 2 ? 2 * m->size : slot * m->size + rank) * (size_t)m->n_max * 4;
}
uint64_t lb_comm_slot_ptr(const lb_comm* m, int slot) { return (uint64_t)m->buf + lb_comm_partial_offset(m, slot, m->rank); }
