"""Tensor-parallel plumbing: exchange buffers (lb_comm_*) and the host-only sharder.

One process per GPU.  The 64-byte IPC handles are passed around by whatever the launcher
has; `make_comm` takes an `all_gather(bytes) -> list[bytes]` callable (torch.distributed's
all_gather_object does the job)."""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import Context, lib, LB_OK
from .model import ModelCfg, WS_SLOTS


def _sigs():
    L = lib()
    vp, i32 = C.c_void_p, C.c_int
    L.lb_comm_create.argtypes = [vp, i32, i32, i32, C.POINTER(vp)]
    L.lb_comm_handle.argtypes = [vp, vp]
    L.lb_comm_open.argtypes = [vp, vp]
    L.lb_comm_set_peer.argtypes = [vp, i32, C.c_uint64]
    L.lb_comm_buffer.argtypes = [vp]
    L.lb_comm_buffer.restype = C.c_uint64
    L.lb_comm_bytes.argtypes = [vp]
    L.lb_comm_bytes.restype = C.c_size_t
    L.lb_comm_partial_offset.argtypes = [vp, i32, i32]
    L.lb_comm_partial_offset.restype = C.c_size_t
    L.lb_comm_flags_offset.argtypes = [vp]
    L.lb_comm_flags_offset.restype = C.c_size_t
    L.lb_comm_allreduce.argtypes = [vp, C.c_uint64, i32, i32]
    L.lb_comm_destroy.argtypes = [vp]
    L.lb_comm_destroy.restype = None
    L.lb_model_set_comm.argtypes = [vp, vp]
    L.lb_model_shard_host.argtypes = [C.POINTER(ModelCfg), i32, i32, i32, i32, C.POINTER(vp), vp, vp, vp,
                                      C.POINTER(i32), C.POINTER(i32)]


class Comm:
    def __init__(self, ctx: Context, rank: int, size: int, n_max: int):
        _sigs()
        self.ctx, self.rank, self.size = ctx, rank, size
        self.h = C.c_void_p(None)
        ctx._check(lib().lb_comm_create(ctx.h, rank, size, n_max, C.byref(self.h)))

    def handle(self) -> bytes:
        buf = C.create_string_buffer(64)
        self.ctx._check(lib().lb_comm_handle(self.h, buf))
        return buf.raw

    def open(self, handles):
        blob = b"".join(handles)
        assert len(blob) == 64 * self.size
        self.ctx._check(lib().lb_comm_open(self.h, C.c_char_p(blob)))

    def set_peer(self, rank: int, buffer_ptr: int):
        """a peer whose exchange buffer this process can address directly (no IPC handle)"""
        self.ctx._check(lib().lb_comm_set_peer(self.h, rank, buffer_ptr))

    @property
    def buffer(self) -> int:
        return lib().lb_comm_buffer(self.h)

    @property
    def nbytes(self) -> int:
        return lib().lb_comm_bytes(self.h)

    def partial_offset(self, slot: int, rank: int) -> int:
        """byte offset, inside any rank's exchange buffer, of `rank`'s partial vector of exchange slot 0 / 1"""
        return lib().lb_comm_partial_offset(self.h, slot, rank)

    @property
    def flags_offset(self) -> int:
        return lib().lb_comm_flags_offset(self.h)

    def allreduce(self, x, n: int, slot: int = 0):
        """x[0..n) += sum over ranks of the partial vectors in `slot` of every rank's buffer (one stand-alone exchange)"""
        self.ctx._check(lib().lb_comm_allreduce(self.h, x.ptr, n, slot))

    def close(self):
        if self.h:
            lib().lb_comm_destroy(self.h)
            self.h = None


def make_comm(ctx: Context, rank: int, size: int, n_max: int, all_gather) -> Comm:
    comm = Comm(ctx, rank, size, n_max)
    if size > 1:
        comm.open(all_gather(comm.handle()))
    return comm


def attach(model, comm: Comm):
    _sigs()
    model.ctx._check(lib().lb_model_set_comm(model.h, comm.h))


def shard_host(cfg: ModelCfg, tp_rank: int, tp_size: int, layer: int, which: int, slots):
    """(qweight [K/8,N], scales [K/128,N], qzeros [K/128,N/8], K, N) of device matrix `which`
    (0 fused input projections, 1 out/o projection, 2 gate|up interleaved, 3 down) for one shard."""
    _sigs()
    arr = (C.c_void_p * WS_SLOTS)(*[(a.ctypes.data if a is not None else None) for a in slots])
    K, N = C.c_int(0), C.c_int(0)
    st = lib().lb_model_shard_host(C.byref(cfg), tp_rank, tp_size, layer, which, arr, None, None, None, C.byref(K), C.byref(N))
    if st != LB_OK:
        raise ValueError(f"shard_host: status {st}")
    K, N = K.value, N.value
    qw = np.empty((K // 8, N), np.uint32)
    sc = np.empty((K // 128, N), np.float16)
    qz = np.empty((K // 128, N // 8), np.uint32)
    st = lib().lb_model_shard_host(C.byref(cfg), tp_rank, tp_size, layer, which, arr, qw.ctypes.data_as(C.c_void_p),
                                   sc.ctypes.data_as(C.c_void_p), qz.ctypes.data_as(C.c_void_p), None, None)
    if st != LB_OK:
        raise ValueError(f"shard_host: status {st}")
    return qw, sc, qz, K, N
