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
