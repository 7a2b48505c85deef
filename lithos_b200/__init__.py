"""lithos_b200 — Python binding (ctypes) of liblithos_b200.so.

The product is the C-ABI shared library declared in ``include/lithos_b200.h``
plus the sm_100a kernel images under ``lithos_b200/kernels``; this module only
loads it and gives the calls Pythonic argument handling (numpy arrays in, numpy
arrays out).  There is no fallback of any kind: if the library, the kernel
images, the CUDA driver or the GPU is missing, the call raises ``LithosError``.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
_LIB_PATH = _HERE / "liblithos_b200.so"
_SRC_DIR = _HERE / "csrc"

# ---- status codes (include/lithos_b200.h) ---------------------------------
LB_OK, LB_ERR_INVALID, LB_ERR_NO_DRIVER, LB_ERR_CUDA, LB_ERR_NO_KERNEL = 0, 1, 2, 3, 4
LB_ERR_DEVICE_WAIT, LB_ERR_IO, LB_ERR_NOMEM, LB_ERR_STATE = 5, 6, 7, 8

GEMV_X_F32, GEMV_Y_F32, GEMV_Y_ACCUM, GEMV_Y_SWIGLU = 1, 2, 4, 8
GEMM_MMA_SYNC, GEMM_TCGEN05 = 16, 32
X_F16, X_F32, X_F32_RMSNORM, X_F32_HEADNORM_SILU = 0, 1, 2, 3
Y_F16, Y_F32, Y_F32_ACCUM, Y_SWIGLU_F16 = 0, 1, 2, 3


class LithosError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"lithos_b200 status {status}: {message}")
        self.status = status


def build(verbose: bool = False) -> None:
    """Compile the host library and every kernel image in-tree (make)."""
    r = subprocess.run(["make", "-C", str(_SRC_DIR), "-j8"], capture_output=True, text=True)
    if verbose or r.returncode != 0:
        print(r.stdout[-4000:])
        print(r.stderr[-4000:])
    if r.returncode != 0:
        raise RuntimeError("building liblithos_b200 failed")


_lib = None


def lib() -> C.CDLL:
    """The loaded shared library (with argument types declared)."""
    global _lib
    if _lib is not None:
        return _lib
    if not _LIB_PATH.exists():
        raise LithosError(LB_ERR_NO_KERNEL, f"{_LIB_PATH} is not built (run lithos_b200.build())")
    L = C.CDLL(str(_LIB_PATH))
    u64, i32, f32, vp, sz = C.c_uint64, C.c_int, C.c_float, C.c_void_p, C.c_size_t
    P = C.POINTER

    def sig(name, res, *args):
        fn = getattr(L, name)
        fn.restype = res
        fn.argtypes = list(args)

    sig("lb_status_string", C.c_char_p, i32)
    sig("lb_version", C.c_char_p)
    sig("lb_init", i32, i32, C.c_char_p, P(vp))
    sig("lb_destroy", None, vp)
    sig("lb_last_error", C.c_char_p, vp)
    sig("lb_device_sm_count", i32, vp)
    sig("lb_device_status", i32, vp, P(C.c_uint32))
    sig("lb_reset_status", i32, vp)
    sig("lb_set_wait_limit", i32, vp, u64)
    sig("lb_launch_count", u64, vp)
    sig("lb_launch_count_reset", None, vp)
    sig("lb_set_pdl", None, vp, i32)
    sig("lb_graph_begin_capture", i32, vp)
    sig("lb_graph_end_capture", i32, vp, P(vp))
    sig("lb_graph_launch", i32, vp, vp)
    sig("lb_graph_kernel_count", i32, vp)
    sig("lb_graph_destroy", None, vp, vp)
    sig("lb_malloc", i32, vp, sz, P(u64))
    sig("lb_free", i32, vp, u64)
    sig("lb_malloc_host", i32, vp, sz, P(vp))
    sig("lb_free_host", i32, vp, vp)
    sig("lb_memcpy_h2d", i32, vp, u64, vp, sz)
    sig("lb_memcpy_d2h", i32, vp, vp, u64, sz)
    sig("lb_memcpy_d2d", i32, vp, u64, u64, sz)
    sig("lb_memset", i32, vp, u64, i32, sz)
    sig("lb_sync", i32, vp)
    sig("lb_timer_start", i32, vp)
    sig("lb_timer_stop", i32, vp, P(f32))
    sig("lb_flush_l2", i32, vp)
    for name in ("lb_fill_u32", "lb_fill_scales_f16"):
        sig(name, None, vp, sz, u64, u64)
    for name in ("lb_fill_normal_f32", "lb_fill_normal_f16", "lb_fill_normal_bf16", "lb_fill_uniform_f32"):
        sig(name, None, vp, sz, u64, u64, f32, f32)
    for name in ("lb_convert_f32_to_f16", "lb_convert_f32_to_bf16", "lb_convert_f16_to_f32", "lb_convert_bf16_to_f32"):
        sig(name, None, vp, vp, sz)
    sig("lb_gemv_int4", i32, vp, u64, u64, u64, u64, u64, i32, i32, i32)
    sig("lb_gemv_int4_host", i32, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32)
    sig("lb_gemv_int4_fused", i32, vp, u64, u64, u64, u64, u64, i32, i32, i32, i32, u64, u64, u64, f32)
    sig("lb_gemv_chain", i32, vp, P(GemvOp), i32)
    sig("lb_gemv_chain_supports", i32, vp, i32, i32, i32)
    sig("lb_gemv_packed_bytes", sz, i32, i32)
    sig("lb_gemv_pack", i32, vp, u64, u64, u64, i32, i32, i32, u64)
    sig("lb_set_chain_reserve", None, vp, i32)
    sig("lb_set_chain_timeline", None, vp, u64)
    sig("lb_set_chain_mailbox", None, vp, i32)
    sig("lb_gemv_packed_copy", u64, vp, u64, i32, i32, i32)
    sig("lb_gemv_pack_version", i32)
    sig("lb_gptq_dequant", i32, vp, u64, u64, u64, u64, i32, i32)
    sig("lb_gemm_int4", i32, vp, u64, u64, u64, u64, u64, i32, i32, i32, i32)
    sig("lb_gptq_unpack", i32, vp, u64, u64, i32, i32)
    sig("lb_dense_bf16_gemv", i32, vp, u64, u64, u64, i32, i32, i32)
    sig("lb_deltanet_step", i32, vp, u64, u64, u64, u64, u64, u64, u64, u64, i32, i32, i32, i32)
    sig("lb_decay_gate", i32, vp, u64, u64, u64, u64, u64, u64, i32)
    sig("lb_attention_decode", i32, vp, u64, u64, u64, u64, u64, u64, u64, u64, u64, i32, i32, i32, i32, i32, f32, f32)
    sig("lb_rmsnorm", i32, vp, u64, u64, u64, u64, u64, i32, i32, f32, i32)
    sig("lb_argmax", i32, vp, u64, i32, u64)
    sig("lb_embed", i32, vp, u64, u64, u64, i32)
    sig("lb_sample_topk", i32, vp, u64, i32, f32, i32, u64, u64, u64, u64, u64)
    _lib = L
    return L


class GemvOp(C.Structure):
    """lb_gemv_op (include/lithos_b200.h): one entry of a GEMV chain"""
    _fields_ = [(n, C.c_uint64) for n in ("packed", "x", "y", "aux0", "aux1", "x_out")] + \
               [(n, C.c_int32) for n in ("K", "N", "x_mode", "y_mode")] + [("eps", C.c_float), ("reserved", C.c_int32)]


# ---- seeded synthetic tensors (host) -----------------------------------------
def _ptr(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


def fill_u32(n: int, seed: int, stream: int) -> np.ndarray:
    out = np.empty(n, dtype=np.uint32)
    lib().lb_fill_u32(_ptr(out), n, seed, stream)
    return out


def fill_scales_f16(n: int, seed: int, stream: int) -> np.ndarray:
    out = np.empty(n, dtype=np.float16)
    lib().lb_fill_scales_f16(_ptr(out), n, seed, stream)
    return out


def fill_normal(n: int, seed: int, stream: int, mean=0.0, std=1.0, dtype="f32") -> np.ndarray:
    """dtype: 'f32' -> float32, 'f16' -> float16, 'bf16' -> uint16 holding bf16 bits."""
    if dtype == "f32":
        out = np.empty(n, dtype=np.float32)
        lib().lb_fill_normal_f32(_ptr(out), n, seed, stream, mean, std)
    elif dtype == "f16":
        out = np.empty(n, dtype=np.float16)
        lib().lb_fill_normal_f16(_ptr(out), n, seed, stream, mean, std)
    elif dtype == "bf16":
        out = np.empty(n, dtype=np.uint16)
        lib().lb_fill_normal_bf16(_ptr(out), n, seed, stream, mean, std)
    else:
        raise ValueError(dtype)
    return out


def fill_uniform(n: int, seed: int, stream: int, lo: float, hi: float) -> np.ndarray:
    out = np.empty(n, dtype=np.float32)
    lib().lb_fill_uniform_f32(_ptr(out), n, seed, stream, lo, hi)
    return out


def f32_to_bf16(a: np.ndarray) -> np.ndarray:
    a = np.ascontiguousarray(a, dtype=np.float32)
    out = np.empty(a.shape, dtype=np.uint16)
    lib().lb_convert_f32_to_bf16(_ptr(a), _ptr(out), a.size)
    return out


def bf16_to_f32(a: np.ndarray) -> np.ndarray:
    a = np.ascontiguousarray(a, dtype=np.uint16)
    return (a.astype(np.uint32) << 16).view(np.float32)


# ---- context -------------------------------------------------------------------
class DeviceBuffer:
    """A device allocation owned by a Context; .ptr is the CUdeviceptr."""

    def __init__(self, ctx: "Context", nbytes: int):
        self.ctx, self.nbytes = ctx, int(nbytes)
        p = C.c_uint64(0)
        ctx._check(lib().lb_malloc(ctx.h, self.nbytes, C.byref(p)))
        self.ptr = p.value

    def upload(self, a: np.ndarray) -> "DeviceBuffer":
        a = np.ascontiguousarray(a)
        assert a.nbytes <= self.nbytes, (a.nbytes, self.nbytes)
        self.ctx._check(lib().lb_memcpy_h2d(self.ctx.h, self.ptr, _ptr(a), a.nbytes))
        self.ctx.sync()  # the source array may be freed by the caller afterwards
        return self

    def download(self, dtype, count: int | None = None, offset_bytes: int = 0) -> np.ndarray:
        dt = np.dtype(dtype)
        n = (self.nbytes - offset_bytes) // dt.itemsize if count is None else count
        out = np.empty(n, dtype=dt)
        self.ctx._check(lib().lb_memcpy_d2h(self.ctx.h, _ptr(out), self.ptr + offset_bytes, out.nbytes))
        self.ctx.sync()
        return out

    def zero(self) -> "DeviceBuffer":
        self.ctx._check(lib().lb_memset(self.ctx.h, self.ptr, 0, self.nbytes))
        return self

    def free(self):
        if self.ptr:
            lib().lb_free(self.ctx.h, self.ptr)
            self.ptr = 0


class Graph:
    """A captured sequence of launches, replayed with one submission."""

    def __init__(self, ctx: "Context", h):
        self.ctx, self.h = ctx, h

    @property
    def kernels(self) -> int:
        return lib().lb_graph_kernel_count(self.h)

    def launch(self):
        self.ctx._check(lib().lb_graph_launch(self.ctx.h, self.h))

    def destroy(self):
        if self.h:
            lib().lb_graph_destroy(self.ctx.h, self.h)
            self.h = None


class Context:
    """One GPU, one stream: the host-side owner of every buffer and launch."""

    def __init__(self, device: int = 0, kernel_dir: str | None = None):
        self.h = C.c_void_p(None)
        st = lib().lb_init(device, kernel_dir.encode() if kernel_dir else None, C.byref(self.h))
        if st != LB_OK:
            msg = lib().lb_last_error(self.h).decode() if self.h else lib().lb_status_string(st).decode()
            if self.h:
                lib().lb_destroy(self.h)
            self.h = None
            raise LithosError(st, msg)
        self.device = device

    def _check(self, st: int):
        if st != LB_OK:
            raise LithosError(st, lib().lb_last_error(self.h).decode())

    def close(self):
        if self.h:
            lib().lb_destroy(self.h)
            self.h = None

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()

    # -- memory --
    def alloc(self, nbytes: int) -> DeviceBuffer:
        return DeviceBuffer(self, nbytes)

    def to_device(self, a: np.ndarray) -> DeviceBuffer:
        a = np.ascontiguousarray(a)
        return DeviceBuffer(self, max(a.nbytes, 16)).upload(a)

    def sync(self):
        self._check(lib().lb_sync(self.h))

    def device_status(self) -> int:
        s = C.c_uint32(0)
        self._check(lib().lb_device_status(self.h, C.byref(s)))
        return s.value

    def reset_status(self):
        self._check(lib().lb_reset_status(self.h))

    def set_wait_limit(self, ns: int):
        """time limit of the kernels' waits on other CTAs / GPUs, nanoseconds (0 = the built-in 2 s)"""
        self._check(lib().lb_set_wait_limit(self.h, int(ns)))

    @property
    def sm_count(self) -> int:
        return lib().lb_device_sm_count(self.h)

    @property
    def launches(self) -> int:
        return lib().lb_launch_count(self.h)

    def reset_launches(self):
        lib().lb_launch_count_reset(self.h)

    def set_chain_mailbox(self, on: bool):
        """hand vectors between consecutive GEMVs of a chain through tagged words (default) or through a grid barrier"""
        lib().lb_set_chain_mailbox(self.h, 1 if on else 0)

    def set_pdl(self, on: bool):
        lib().lb_set_pdl(self.h, 1 if on else 0)

    # -- graphs --
    def begin_capture(self):
        self._check(lib().lb_graph_begin_capture(self.h))

    def end_capture(self) -> "Graph":
        g = C.c_void_p(None)
        self._check(lib().lb_graph_end_capture(self.h, C.byref(g)))
        return Graph(self, g)

    # -- timing --
    def timer_start(self):
        self._check(lib().lb_timer_start(self.h))

    def timer_stop(self) -> float:
        ms = C.c_float(0)
        self._check(lib().lb_timer_stop(self.h, C.byref(ms)))
        return ms.value

    def flush_l2(self):
        self._check(lib().lb_flush_l2(self.h))

    # -- ops (device pointers) --
    def gemv_int4(self, qweight, scales, qzeros, x, y, K, N, flags=0):
        self._check(lib().lb_gemv_int4(self.h, qweight.ptr, scales.ptr, qzeros.ptr if qzeros else 0, x.ptr, y.ptr, K, N, flags))

    def gemv_int4_fused(self, qweight, scales, qzeros, x, y, K, N, x_mode, y_mode, aux0=None, aux1=None, x_out=None, eps=1e-6):
        self._check(lib().lb_gemv_int4_fused(self.h, qweight.ptr, scales.ptr, qzeros.ptr if qzeros else 0, x.ptr, y.ptr, K, N,
                                             x_mode, y_mode, aux0.ptr if aux0 else 0, aux1.ptr if aux1 else 0,
                                             x_out.ptr if x_out else 0, eps))

    def gemv_pack(self, qweight, scales, qzeros, K, N, swiglu=False) -> "DeviceBuffer":
        """strip-packed copy of a reference-format matrix for gemv_chain (device to device, once per matrix)"""
        out = self.alloc(lib().lb_gemv_packed_bytes(K, N))
        self._check(lib().lb_gemv_pack(self.h, qweight.ptr, scales.ptr, qzeros.ptr if qzeros else 0, K, N, 1 if swiglu else 0, out.ptr))
        return out

    def gemv_packed_copy(self, qweight, K, N, swiglu=False) -> int:
        """device address of the strip-packed copy gemv_int4 reads for this matrix, or 0"""
        return lib().lb_gemv_packed_copy(self.h, qweight.ptr, K, N, 1 if swiglu else 0)

    def gemv_chain(self, ops):
        """ops: dicts (packed, x, y, K, N, x_mode, y_mode, aux0, aux1, x_out, eps); all of them run as ONE persistent launch"""
        arr = (GemvOp * len(ops))()
        for a, o in zip(arr, ops):
            for name in ("packed", "x", "y", "aux0", "aux1", "x_out"):
                b = o.get(name)
                setattr(a, name, b.ptr if b else 0)
            a.K, a.N, a.x_mode, a.y_mode, a.eps = o["K"], o["N"], o["x_mode"], o["y_mode"], o.get("eps", 1e-6)
        self._check(lib().lb_gemv_chain(self.h, arr, len(ops)))

    def gemv_chain_supports(self, K, N, swiglu=False) -> bool:
        return lib().lb_gemv_chain_supports(self.h, K, N, 1 if swiglu else 0) == 0

    def gemv_int4_host(self, qweight, scales, qzeros, x, y, K, N, flags=0, weights_resident=False):
        self._check(lib().lb_gemv_int4_host(self.h, _ptr(qweight), _ptr(scales), _ptr(qzeros) if qzeros is not None else None,
                                            _ptr(x), _ptr(y), K, N, flags, 1 if weights_resident else 0))

    def gemm_int4(self, qweight, scales, qzeros, x, y, K, N, B, flags=0):
        """Y[B,N] = X[B,K] W for up to 64 tokens; the weights are read once for the whole batch."""
        self._check(lib().lb_gemm_int4(self.h, qweight.ptr, scales.ptr, qzeros.ptr if qzeros else 0, x.ptr, y.ptr, K, N, B, flags))

    def gptq_dequant(self, qweight, scales, qzeros, w_out, K, N):
        self._check(lib().lb_gptq_dequant(self.h, qweight.ptr, scales.ptr, qzeros.ptr if qzeros else 0, w_out.ptr, K, N))

    def gptq_unpack(self, qweight, q_out, K, N):
        self._check(lib().lb_gptq_unpack(self.h, qweight.ptr, q_out.ptr, K, N))

    def dense_bf16_gemv(self, w, x, y, N, K, x_is_f32=False):
        self._check(lib().lb_dense_bf16_gemv(self.h, w.ptr, x.ptr, y.ptr, N, K, 1 if x_is_f32 else 0))

    def deltanet_step(self, state, q, k, v, z, g, beta, out, HV, HK, n_steps=1, in_is_f32=False):
        self._check(lib().lb_deltanet_step(self.h, state.ptr, q.ptr, k.ptr, v.ptr, z.ptr if z else 0, g.ptr, beta.ptr, out.ptr,
                                           HV, HK, n_steps, 1 if in_is_f32 else 0))

    def decay_gate(self, a, a_log, dt_bias, b, g_out, beta_out, n):
        self._check(lib().lb_decay_gate(self.h, a.ptr, a_log.ptr, dt_bias.ptr, b.ptr if b else 0, g_out.ptr,
                                        beta_out.ptr if beta_out else 0, n))

    def attention_decode(self, q, k_new, v_new, gate, q_norm_w, k_norm_w, k_cache, v_cache, out, pos, HQ, HKV,
                         in_is_f32=False, rot_dims=64, rope_theta=1e7, eps=1e-6):
        self._check(lib().lb_attention_decode(self.h, q.ptr, k_new.ptr, v_new.ptr, gate.ptr if gate else 0,
                                              q_norm_w.ptr if q_norm_w else 0, k_norm_w.ptr if k_norm_w else 0,
                                              k_cache.ptr, v_cache.ptr, out.ptr, pos, HQ, HKV, 1 if in_is_f32 else 0,
                                              rot_dims, rope_theta, eps))

    def rmsnorm(self, x, res, w, y, sum_out, rows, D, eps=1e-6, one_plus_w=True):
        self._check(lib().lb_rmsnorm(self.h, x.ptr, res.ptr if res else 0, w.ptr, y.ptr, sum_out.ptr if sum_out else 0,
                                     rows, D, eps, 1 if one_plus_w else 0))

    def argmax(self, x, n, out_idx):
        self._check(lib().lb_argmax(self.h, x.ptr, n, out_idx.ptr))

    def sample_topk(self, x, n, temperature, top_k, seed, counter, out_idx, probs_out=None, idx_out=None):
        self._check(lib().lb_sample_topk(self.h, x.ptr, n, temperature, top_k, seed, counter, out_idx.ptr,
                                         probs_out.ptr if probs_out else 0, idx_out.ptr if idx_out else 0))

    def embed(self, table, token, out, D):
        self._check(lib().lb_embed(self.h, table.ptr, token.ptr, out.ptr, D))
