"""Drop-in cubins (lithos_b200/kernels/compat/): each is loaded and launched the way the reference
launcher does it -- file name, entry symbol, positional parameter block, grid and block from
src/launcher.s -- through lb_module_load / lb_module_get_kernel / lb_launch_kernel, and compared
with the oracle (fp32 element-wise kernels: within a few ulp; reductions: 1e-5 relative)."""
import ctypes as C
from pathlib import Path

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
_FN = {}
COMPAT = Path(__file__).resolve().parent.parent / "lithos_b200" / "kernels" / "compat"


def launch(ctx, lb, name, entry, vals, grid, block, smem=0):
    L = lb.lib()
    L.lb_module_load.argtypes = [C.c_void_p, C.c_char_p, C.POINTER(C.c_int)]
    L.lb_module_get_kernel.argtypes = [C.c_void_p, C.c_int, C.c_char_p, C.POINTER(C.c_uint64)]
    L.lb_launch_kernel.argtypes = [C.c_void_p, C.c_uint64] + [C.c_uint] * 7 + [C.POINTER(C.c_void_p)]
    fn = _FN.get((id(ctx), name, entry))
    if fn is None:              # load each image once per context, as the launcher does at start-up
        mod, fn = C.c_int(), C.c_uint64()
        ctx._check(L.lb_module_load(ctx.h, str(COMPAT / name).encode(), C.byref(mod)))
        ctx._check(L.lb_module_get_kernel(ctx.h, mod, entry.encode(), C.byref(fn)))
        _FN[(id(ctx), name, entry)] = fn
    params = (C.c_void_p * len(vals))(*[C.cast(C.pointer(v), C.c_void_p) for v in vals])
    ctx._check(L.lb_launch_kernel(ctx.h, fn, grid, 1, 1, block, 1, 1, smem, params))
    ctx.sync()
    assert ctx.device_status() == 0


def u64(b):
    return C.c_uint64(b.ptr)


def test_embed_f16(ctx, lb):
    rng = np.random.default_rng(1)
    table = rng.standard_normal((64, 5120)).astype(np.float16)
    d_t, d_o = ctx.to_device(table), ctx.alloc(5120 * 4)
    for tok in (0, 17, 63):
        launch(ctx, lb, "embed_f16.cubin", "embed_f16", [C.c_uint32(tok), u64(d_t), u64(d_o)], 5, 256)
        assert np.array_equal(d_o.download(np.float32, 5120), table[tok].astype(np.float32))


def test_norm(ctx, lb, oracle):
    rng = np.random.default_rng(2)
    D = 5120
    x, r = rng.standard_normal(D).astype(np.float32), rng.standard_normal(D).astype(np.float32)
    w = oracle.f32_to_bf16(rng.standard_normal(D).astype(np.float32))
    d_x, d_r, d_w, d_y = ctx.to_device(x), ctx.to_device(r), ctx.to_device(w), ctx.alloc(D * 4)
    launch(ctx, lb, "norm.cubin", "norm", [u64(d_x), u64(d_r), u64(d_w), u64(d_y), C.c_uint32(D), C.c_float(1e-6)], 1, 256)
    want, _ = oracle.rmsnorm(x, oracle.bf16_to_f32(w), res=r, eps=1e-6, one_plus_w=False)
    np.testing.assert_allclose(d_y.download(np.float32, D), want, rtol=1e-5, atol=1e-6)


def test_activate_and_gate_sigmoid(ctx, lb, oracle):
    rng = np.random.default_rng(3)
    n = 17408
    g, u = rng.standard_normal(n).astype(np.float32) * 3, rng.standard_normal(n).astype(np.float32)
    d_g, d_u, d_o = ctx.to_device(g), ctx.to_device(u), ctx.alloc(n * 4)
    launch(ctx, lb, "activate.cubin", "activate", [u64(d_g), u64(d_u), u64(d_o), C.c_uint32(n)], 68, 256)
    np.testing.assert_allclose(d_o.download(np.float32, n), oracle.swiglu(g, u), rtol=2e-6, atol=1e-7)
    n = 6144
    o, z = rng.standard_normal(n).astype(np.float32), rng.standard_normal(n).astype(np.float32) * 4
    d_o2, d_z = ctx.to_device(o), ctx.to_device(z)
    launch(ctx, lb, "gate_sigmoid.cubin", "gate_sigmoid", [u64(d_o2), u64(d_z), C.c_uint32(n)], 24, 256)
    want = (o.astype(np.float64) / (1.0 + np.exp(-z.astype(np.float64)))).astype(np.float32)
    np.testing.assert_allclose(d_o2.download(np.float32, n), want, rtol=2e-6, atol=1e-7)


def test_l2norm(ctx, lb, oracle):
    rng = np.random.default_rng(4)
    for D in (128, 2048):
        x = rng.standard_normal(D).astype(np.float32)
        d_x = ctx.to_device(x)
        launch(ctx, lb, "reduce.cubin", "l2norm", [u64(d_x), u64(d_x), C.c_uint32(D)], 1, 256)   # in place, as launched
        np.testing.assert_allclose(d_x.download(np.float32, D), oracle.l2norm(x), rtol=1e-5, atol=1e-7)


def test_lm_head(ctx, lb):
    rng = np.random.default_rng(5)
    rows, D = 4096, 5120            # the kernel takes its row count from the grid: 4 rows per CTA
    w = (rng.standard_normal((rows, D)) * 0.05).astype(np.float16)
    x = rng.standard_normal(D).astype(np.float32)
    d_w, d_x, d_y = ctx.to_device(w), ctx.to_device(x), ctx.alloc(rows * 4)
    launch(ctx, lb, "lm_head.cubin", "lm_head", [u64(d_w), u64(d_x), u64(d_y)], rows // 4, 128)
    want = w.astype(np.float64) @ x.astype(np.float64)
    got = d_y.download(np.float32, rows)
    assert np.max(np.abs(got - want)) <= 1e-5 * np.max(np.abs(want)) + 1e-5
    assert int(np.argmax(got)) == int(np.argmax(want))


def test_sample(ctx, lb):
    """entry sample: arg-max of logits / temperature, the first maximum wins; top_k is read and ignored"""
    rng = np.random.default_rng(8)
    V = 248320
    logits = rng.standard_normal(V).astype(np.float32) * 4
    d_l, d_t = ctx.to_device(logits), ctx.alloc(16)
    for temp, top_k in ((1.0, 1), (0.7, 40), (2.5, 0)):
        launch(ctx, lb, "sample.cubin", "sample", [u64(d_l), u64(d_t), C.c_uint32(V), C.c_float(temp), C.c_uint32(top_k)], 1, 256)
        assert int(d_t.download(np.uint32, 1)[0]) == int(np.argmax(logits))
    # ties: the smallest index among the maxima, wherever they sit
    logits[:] = -1.0
    logits[[200001, 777, 131072, 248319]] = 5.0
    d_l.upload(logits)
    for block in (256, 1024, 96):
        launch(ctx, lb, "sample.cubin", "sample", [u64(d_l), u64(d_t), C.c_uint32(V), C.c_float(1.0), C.c_uint32(1)], 1, block)
        assert int(d_t.download(np.uint32, 1)[0]) == 777
    launch(ctx, lb, "sample.cubin", "sample", [u64(d_l), u64(d_t), C.c_uint32(5), C.c_float(1.0), C.c_uint32(1)], 1, 256)
    assert int(d_t.download(np.uint32, 1)[0]) == 0
    d_l.free()
    d_t.free()


def test_attention_score_three_entries(ctx, lb, oracle):
    """attention_score.cubin: the .ls parameter block on an fp32 and on a bf16 cache, and the launcher's 7-parameter
    block; all against the oracle's soft-max attention (natural exp, -inf start), <= 2e-3 of max|out|"""
    from helpers import attention_case, rel_err_max
    HQ, HKV, L = 24, 4, 777
    c = attention_case(901, L, HQ, HKV)
    f = oracle.bf16_to_f32
    q = f(c["q"]).astype(np.float32)
    want = oracle.attention_decode(q, c["kc"], c["vc"], None, L, HQ, HKV)
    d_q, d_o = ctx.to_device(q), ctx.alloc(HQ * 256 * 4)
    kc32, vc32 = ctx.to_device(f(c["kc"])), ctx.to_device(f(c["vc"]))
    kc16, vc16 = ctx.to_device(c["kc"]), ctx.to_device(c["vc"])
    ls_block = lambda k, v, seq, cur: [u64(d_q), u64(k), u64(v), u64(d_o), C.c_uint32(256), C.c_uint32(seq), C.c_uint32(cur),
                                       C.c_uint32(HKV), C.c_uint32(HQ)]
    launch(ctx, lb, "attention_score.cubin", "attention_score", ls_block(kc32, vc32, L, L), HQ, 256)
    assert rel_err_max(d_o.download(np.float32, HQ * 256), want.ravel()) <= 2e-3
    d_o.zero()
    launch(ctx, lb, "attention_score.cubin", "attention_score_bf16", ls_block(kc16, vc16, L + 50, L), HQ, 256)   # current_pos bounds it
    assert rel_err_max(d_o.download(np.float32, HQ * 256), want.ravel()) <= 2e-3
    d_o.zero()
    launch(ctx, lb, "attention_score.cubin", "attention_score_launcher",
           [u64(d_q), u64(kc32), u64(vc32), u64(d_o), C.c_uint32(L), C.c_uint32(256), C.c_uint32(HQ)], 24, 256)
    assert rel_err_max(d_o.download(np.float32, HQ * 256), want.ravel()) <= 2e-3
    # one attended row: the output is that row of V
    launch(ctx, lb, "attention_score.cubin", "attention_score", ls_block(kc32, vc32, 1, 1), HQ, 256)
    v0 = np.repeat(f(c["vc"])[0], HQ // HKV, axis=0)
    np.testing.assert_allclose(d_o.download(np.float32, HQ * 256).reshape(HQ, 256), v0, rtol=1e-6, atol=0)


def test_recur_deltanet_fused_and_launcher_alias(ctx, lb, oracle):
    """recur.cubin: deltanet_fused with the .ls parameter block, 16 key heads x 3, three tokens, against the oracle
    (which the fixture computed from the reference's kernel text pins); deltanet_step with the launcher's block"""
    from helpers import rel_err_max
    HK, G, T = 16, 3, 3
    HV = HK * G
    rng = np.random.default_rng(5)
    state = (rng.standard_normal((HV, 128, 128)) * 0.02).astype(np.float32)
    d_state = ctx.to_device(state)
    d_out = ctx.alloc(HV * 128 * 4)
    ref = state.copy()
    for t in range(T):
        q = rng.standard_normal((HK, 128)).astype(np.float32)
        k = rng.standard_normal((HK, 128)).astype(np.float32)
        q /= np.linalg.norm(q, axis=1, keepdims=True) * np.sqrt(128.0)
        k /= np.linalg.norm(k, axis=1, keepdims=True)
        v, z = rng.standard_normal((HV, 128)).astype(np.float32), rng.standard_normal((HV, 128)).astype(np.float32)
        g, b = rng.uniform(0.3, 1.0, HV).astype(np.float32), rng.uniform(0.1, 0.9, HV).astype(np.float32)
        want = oracle.deltanet_step(ref, q, k, v, z, g, b, HV, HK)
        bufs = [ctx.to_device(a) for a in (q, k, v, z, g, b)]
        launch(ctx, lb, "recur.cubin", "deltanet_fused", [u64(x) for x in bufs] + [u64(d_state), u64(d_out), C.c_uint32(128), C.c_uint32(G)], HK, 128)
        assert rel_err_max(d_out.download(np.float32, HV * 128), want.ravel()) <= 1e-4
    got = d_state.download(np.float32, HV * 128 * 128).reshape(HV, -1).astype(np.float64)
    fro = np.linalg.norm(got - ref.reshape(HV, -1), axis=1) / np.linalg.norm(ref.reshape(HV, -1), axis=1)
    assert fro.max() <= 1e-5
    # the launcher's element-wise placeholder: state += value * key; output = query * state
    n = 2048
    s, qq, kk, vv = (rng.standard_normal(n).astype(np.float32) for _ in range(4))
    d = [ctx.to_device(a) for a in (s, qq, kk, vv)]
    d_o = ctx.alloc(n * 4)
    launch(ctx, lb, "recur.cubin", "deltanet_step", [u64(d[0]), u64(d[1]), u64(d[1]), u64(d[2]), u64(d[3]), u64(d_o), C.c_uint32(n)], 8, 256)
    s2 = (vv.astype(np.float64) * kk + s).astype(np.float32)
    np.testing.assert_allclose(d[0].download(np.float32, n), s2, rtol=1e-6, atol=1e-7)
    np.testing.assert_allclose(d_o.download(np.float32, n), qq * s2, rtol=1e-6, atol=1e-7)


def test_conv1d_three_slices_as_launched(ctx, lb, oracle):
    """conv1d.cubin: Q, K and V slices of a DeltaNet layer's qkv vector, three calls per token as the launcher makes
    them (in place), four tokens, against the oracle's conv1d_step on every slice"""
    rng = np.random.default_rng(6)
    slices = [(16, 128), (16, 128), (48, 128)]
    for heads, ch in slices[1:]:                      # K-sized and V-sized slices (Q is the same shape as K)
        N = heads * ch
        w = (rng.standard_normal((4, N)) * 0.3).astype(np.float32)
        hist = rng.standard_normal((3, N)).astype(np.float32)
        d_w, d_h, d_x = ctx.to_device(w), ctx.to_device(hist), ctx.alloc(N * 4)
        d_wb = ctx.to_device(oracle.f32_to_bf16(w))
        d_h2, d_x2 = ctx.to_device(hist), ctx.alloc(N * 4)
        h_ref, h_ref2 = hist.copy(), hist.copy()
        wb = oracle.bf16_to_f32(oracle.f32_to_bf16(w)).reshape(4, N)
        for t in range(4):
            x = rng.standard_normal(N).astype(np.float32)
            d_x.upload(x)
            d_x2.upload(x)
            launch(ctx, lb, "conv1d.cubin", "conv1d", [u64(d_x), u64(d_w), u64(d_h), u64(d_x), C.c_uint32(heads), C.c_uint32(ch)], (N + 255) // 256, 256)
            y, h_ref = oracle.conv1d_step(x, w, h_ref)
            np.testing.assert_allclose(d_x.download(np.float32, N), y, rtol=1e-6, atol=1e-6)
            launch(ctx, lb, "conv1d.cubin", "conv1d_bf16w", [u64(d_x2), u64(d_wb), u64(d_h2), u64(d_x2), C.c_uint32(heads), C.c_uint32(ch)], (N + 255) // 256, 256)
            y2, h_ref2 = oracle.conv1d_step(x, wb, h_ref2)
            np.testing.assert_allclose(d_x2.download(np.float32, N), y2, rtol=1e-6, atol=1e-6)
        assert np.array_equal(d_h.download(np.float32, 3 * N).reshape(3, N), h_ref)


def test_rotate_table_driven_and_rope_interleaved(ctx, lb, oracle):
    """rotate.cubin: `rotate` with the launcher's block and tables (half-split over 256 dims, theta 1e6, 24 query heads and
    the 4 key heads that follow them); `rope` with the .ls block (interleaved pairs on the first 64 dims, theta 1e7)"""
    rng = np.random.default_rng(7)
    HQ, HKV, D, NPOS = 24, 4, 256, 64
    cos_t, sin_t = oracle.rope_tables(NPOS, D // 2, 1e6)
    buf = rng.standard_normal((HQ + 2 * HKV, D)).astype(np.float32)      # the launcher's q | k | v slices, back to back
    d_b, d_c, d_s = ctx.to_device(buf), ctx.to_device(cos_t), ctx.to_device(sin_t)
    from lithos_b200 import DeviceBuffer
    k_view = DeviceBuffer.__new__(DeviceBuffer)
    k_view.ctx, k_view.ptr, k_view.nbytes = ctx, d_b.ptr + HQ * D * 4, HKV * D * 4
    pos = 37
    launch(ctx, lb, "rotate.cubin", "rotate", [u64(d_b), u64(k_view), u64(d_c), u64(d_s), C.c_uint32(pos), C.c_uint32(D), C.c_uint32(HQ)], 24, 256)
    got = d_b.download(np.float32, buf.size).reshape(buf.shape)
    np.testing.assert_allclose(got[:HQ], oracle.rotate_half(buf[:HQ], HQ, D, cos_t, sin_t, pos).reshape(HQ, D), rtol=1e-6, atol=1e-6)
    np.testing.assert_allclose(got[HQ:HQ + HKV], oracle.rotate_half(buf[HQ:HQ + HKV], HKV, D, cos_t, sin_t, pos).reshape(HKV, D), rtol=1e-6, atol=1e-6)
    assert np.array_equal(got[HQ + HKV:], buf[HQ + HKV:])               # the V slice behind K is untouched
    for p in (5, 4100):
        q, k = rng.standard_normal((HKV, D)).astype(np.float32), rng.standard_normal((HKV, D)).astype(np.float32)
        d_q, d_k, d_qo, d_ko = ctx.to_device(q), ctx.to_device(k), ctx.alloc(q.nbytes), ctx.alloc(k.nbytes)
        launch(ctx, lb, "rotate.cubin", "rope", [u64(d_q), u64(d_k), u64(d_qo), u64(d_ko), C.c_uint32(D), C.c_uint32(p)], HKV, 128)
        np.testing.assert_allclose(d_qo.download(np.float32, q.size), oracle.rope(q, HKV, D, 64, p, 1e7).ravel(), rtol=0, atol=2e-6 * np.abs(q).max())
        np.testing.assert_allclose(d_ko.download(np.float32, k.size), oracle.rope(k, HKV, D, 64, p, 1e7).ravel(), rtol=0, atol=2e-6 * np.abs(k).max())
