"""GPU: lb_attention_decode_noalloc, the decode-attention entry point for callers that cannot allocate
(their own graph capture, pre-sized real-time loops, plugins inside someone else's memory pool).  Its
scratch is an array inside the library's device image.  Checked through the C ABI against the CPU oracle and
against the regular lb_attention_decode on the same inputs, two calls in a row (the second reuses whatever the
first left in the array), within the tolerance the attention tests use (2e-3 of max|out|).  This file sorts last
on purpose: a run that stops at the first failure has then already run every other test."""
import ctypes as C

import numpy as np
import pytest

from helpers import attention_case, rel_err_max

pytestmark = pytest.mark.gpu


def _device_sync():
    # the entry point runs on the default stream; the context's own stream does not wait for it
    cuda = C.CDLL("libcuda.so.1")
    assert cuda.cuCtxSynchronize() == 0


def test_noalloc_attention_matches_oracle_and_regular_entry_twice(ctx, lb, oracle):
    L_ = lb.lib()
    u64, i32 = C.c_uint64, C.c_int
    L_.lb_attention_decode_noalloc.restype = i32
    L_.lb_attention_decode_noalloc.argtypes = [C.c_void_p] + [u64] * 9 + [i32] * 5 + [C.c_float, C.c_float, C.c_char_p, C.c_size_t]
    HQ, HKV = 24, 4
    err = C.create_string_buffer(256)
    for call, L in enumerate((777, 3000)):          # 12 slices, then the 16-slice cap
        c = attention_case(500 + call, L, HQ, HKV)
        f = oracle.bf16_to_f32
        kc_o, vc_o = c["kc"].copy(), c["vc"].copy()
        want = oracle.attention_step(f(c["q"]), f(c["k_new"]), f(c["v_new"]), f(c["gate"]), f(c["q_norm_w"]),
                                     f(c["k_norm_w"]), kc_o, vc_o, L - 1, HQ, HKV).ravel()
        outs = []
        for which in ("regular", "noalloc"):
            d = {n: ctx.to_device(c[n]) for n in ("q", "k_new", "v_new", "gate", "q_norm_w", "k_norm_w")}
            d_kc, d_vc = ctx.to_device(c["kc"]), ctx.to_device(c["vc"])
            d_out = ctx.alloc(HQ * 256 * 4).zero()
            ctx.sync()
            if which == "regular":
                ctx.attention_decode(d["q"], d["k_new"], d["v_new"], d["gate"], d["q_norm_w"], d["k_norm_w"], d_kc, d_vc,
                                     d_out, L - 1, HQ, HKV)
                ctx.sync()
            else:
                st = L_.lb_attention_decode_noalloc(None, d["q"].ptr, d["k_new"].ptr, d["v_new"].ptr, d["gate"].ptr,
                                                    d["q_norm_w"].ptr, d["k_norm_w"].ptr, d_kc.ptr, d_vc.ptr, d_out.ptr,
                                                    L - 1, HQ, HKV, 0, 64, 1e7, 1e-6, err, 256)
                assert st == lb.LB_OK, err.value.decode()
                _device_sync()
            out = d_out.download(np.float32, HQ * 256)
            k_row = d_kc.download(np.uint16, HKV * 256, offset_bytes=(L - 1) * HKV * 256 * 2)
            outs.append((out, k_row))
            for b in list(d.values()) + [d_kc, d_vc, d_out]:
                b.free()
        assert np.isfinite(outs[1][0]).all()
        assert rel_err_max(outs[1][0], want) <= 2e-3           # the checker of record: the CPU oracle
        assert rel_err_max(outs[1][0], outs[0][0]) <= 2e-3     # and the existing entry point
        kf, kw = f(outs[1][1]), f(kc_o[L - 1].ravel())
        assert np.max(np.abs(kf - kw)) <= 2.0 ** -7 * np.max(np.abs(kw))
        assert np.array_equal(outs[1][1], outs[0][1])       # the appended key row: same arithmetic, same bits


def test_noalloc_rejects_what_does_not_fit(ctx, lb):
    L_ = lb.lib()
    u64, i32 = C.c_uint64, C.c_int
    L_.lb_attention_decode_noalloc.restype = i32
    L_.lb_attention_decode_noalloc.argtypes = [C.c_void_p] + [u64] * 9 + [i32] * 5 + [C.c_float, C.c_float, C.c_char_p, C.c_size_t]
    d = ctx.alloc(1 << 16)
    err = C.create_string_buffer(256)
    # 16 KV heads: beyond the built-in scratch
    st = L_.lb_attention_decode_noalloc(None, d.ptr, d.ptr, d.ptr, 0, 0, 0, d.ptr, d.ptr, d.ptr, 0, 16, 16, 0, 64, 1e7, 1e-6, err, 256)
    assert st == lb.LB_ERR_INVALID and b"8 KV heads" in err.value
    # 8 query heads per KV head: not an instantiated ratio
    st = L_.lb_attention_decode_noalloc(None, d.ptr, d.ptr, d.ptr, 0, 0, 0, d.ptr, d.ptr, d.ptr, 0, 8, 1, 0, 64, 1e7, 1e-6, err, 256)
    assert st == lb.LB_ERR_INVALID
    d.free()


def test_noalloc_attention_inside_a_stream_capture(ctx, lb):
    """What the entry point is for: the caller captures its own CUDA graph (driver API here) with the call inside, then
    replays it.  The call must add only capturable work (a memset of its counters and the kernel) to the caller's stream,
    and every replay must leave the bits of the uncaptured call (same position, so the appended row is rewritten in place)."""
    L_ = lb.lib()
    u64, i32 = C.c_uint64, C.c_int
    L_.lb_attention_decode_noalloc.restype = i32
    L_.lb_attention_decode_noalloc.argtypes = [C.c_void_p] + [u64] * 9 + [i32] * 5 + [C.c_float, C.c_float, C.c_char_p, C.c_size_t]
    cuda = C.CDLL("libcuda.so.1")
    HQ, HKV, L = 24, 4, 1500
    c = attention_case(901, L, HQ, HKV)
    d = {n: ctx.to_device(c[n]) for n in ("q", "k_new", "v_new", "gate", "q_norm_w", "k_norm_w")}
    d_kc, d_vc = ctx.to_device(c["kc"]), ctx.to_device(c["vc"])
    d_out = ctx.alloc(HQ * 256 * 4).zero()
    ctx.sync()
    err = C.create_string_buffer(256)

    def call(stream):
        st = L_.lb_attention_decode_noalloc(stream, d["q"].ptr, d["k_new"].ptr, d["v_new"].ptr, d["gate"].ptr, d["q_norm_w"].ptr,
                                            d["k_norm_w"].ptr, d_kc.ptr, d_vc.ptr, d_out.ptr, L - 1, HQ, HKV, 0, 64, 1e7, 1e-6, err, 256)
        assert st == lb.LB_OK, err.value.decode()

    call(None)                                       # uncaptured (also the call that looks the scratch array up)
    _device_sync()
    want = d_out.download(np.float32, HQ * 256)
    stream, graph, gexec = C.c_void_p(), C.c_void_p(), C.c_void_p()
    assert cuda.cuStreamCreate(C.byref(stream), 1) == 0                      # CU_STREAM_NON_BLOCKING
    assert cuda.cuStreamBeginCapture_v2(stream, 0) == 0                      # CU_STREAM_CAPTURE_MODE_GLOBAL
    call(stream)
    assert cuda.cuStreamEndCapture(stream, C.byref(graph)) == 0 and graph.value
    assert cuda.cuGraphInstantiateWithFlags(C.byref(gexec), graph, C.c_ulonglong(0)) == 0
    for _ in range(2):
        d_out.zero()
        ctx.sync()
        assert cuda.cuGraphLaunch(gexec, stream) == 0
        assert cuda.cuStreamSynchronize(stream) == 0
        assert np.array_equal(d_out.download(np.float32, HQ * 256), want)
    assert cuda.cuGraphExecDestroy(gexec) == 0 and cuda.cuGraphDestroy(graph) == 0 and cuda.cuStreamDestroy_v2(stream) == 0
    for b in list(d.values()) + [d_kc, d_vc, d_out]:
        b.free()
