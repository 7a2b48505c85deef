"""lb_gemv_chain: several fused int4 GEMVs in ONE persistent launch (grid barrier between them).

Oracle comparisons use the GEMV tolerance (max |diff| / max |y| <= 1e-3).  The chain is also
compared with the same GEMVs launched one by one through lb_gemv_int4_fused, run twice (the
barrier words and tile counters must come back to zero; results must be bit-identical run to run)
and replayed from a CUDA graph.
"""
import numpy as np
import pytest

from helpers import gptq_case, rel_err_max

pytestmark = pytest.mark.gpu
TOL = 1e-3


def _op(d, x, y, K, N, x_mode, y_mode, aux0=None, aux1=None, x_out=None):
    """d = [qweight, scales, qzeros, packed]"""
    return dict(qweight=d[0], scales=d[1], qzeros=d[2], packed=d[3], x=x, y=y, K=K, N=N, x_mode=x_mode, y_mode=y_mode, aux0=aux0,
                aux1=aux1, x_out=x_out, eps=1e-6)


def _dev(ctx, qw, sc, qz, K, N, swiglu=False):
    d = [ctx.to_device(qw), ctx.to_device(sc), ctx.to_device(qz) if qz is not None else None]
    d.append(ctx.gemv_pack(d[0], d[1], d[2], K, N, swiglu))
    return d


@pytest.mark.parametrize("K,N,zeros", [(5120, 16384, True), (6144, 5120, True), (17408, 5120, False), (5120, 34816, True),
                                       (1024, 37888, True), (256, 64, True), (640, 2048, True)])
def test_single_gemv_vs_oracle(ctx, lb, oracle, K, N, zeros):
    """the decode step's four shapes, the widest strips (37888 = 148 SMs x 256 columns) and a matrix with
    fewer octets than SMs, as chains of one"""
    qw, sc, qz, x = gptq_case(K, N, seed=21, zeros=zeros)
    want, _ = oracle.gptq_gemv(qw, sc, qz, x, K, N)
    d = _dev(ctx, qw, sc, qz, K, N)
    d_x, d_y = ctx.to_device(x), ctx.alloc(N * 4)
    ctx.gemv_chain([_op(d, d_x, d_y, K, N, lb.X_F16, lb.Y_F32)])
    got = d_y.download(np.float32, N)
    assert ctx.device_status() == 0
    assert rel_err_max(got, want) <= TOL
    for b in d + [d_x, d_y]:
        if b:
            b.free()


@pytest.mark.parametrize("K,N,swiglu,zeros", [(640, 5120, False, True), (256, 4096, True, True), (384, 1184, False, False)])
def test_pack_is_byte_exact(ctx, lb, oracle, K, N, swiglu, zeros):
    """lb_gemv_pack against the numpy restatement of the strip layout: strips of 4 and 5 octets with a trailing single
    (5120 columns over the SMs), SwiGLU pairs, one octet per SM without a zero-point tensor"""
    qw, sc, qz, _ = gptq_case(K, N, seed=31, zeros=zeros)
    d = _dev(ctx, qw, sc, qz, K, N, swiglu)
    got = d[3].download(np.uint32, N // 8 * (K // 128) * 136)
    want = oracle.pack_strips(qw, sc, qz, K, N, ctx.sm_count, swiglu)
    assert np.array_equal(got, want)
    for b in d:
        if b:
            b.free()


def _layer_case(ctx, lb, seed, H=5120, V=6144, I=17408, NIN=16384):
    """the GEMVs between two token mixers: out projection (per-head norm, silu(z) gate, residual add),
    gate/up (RMSNorm, SwiGLU), down (residual add), next layer's input projection (RMSNorm, fp16 copy out)"""
    mats = {"out": gptq_case(V, H, seed + 1), "gu": gptq_case(H, 2 * I, seed + 2), "down": gptq_case(I, H, seed + 3, zeros=False),
            "in": gptq_case(H, NIN, seed + 4)}
    dev = {k: _dev(ctx, m[0], m[1], m[2], m[0].shape[0] * 8, m[0].shape[1], swiglu=(k == "gu")) for k, m in mats.items()}
    host = dict(mix=lb.fill_normal(V, seed, 40, std=2.0), z=lb.fill_normal(V, seed, 41), hw=lb.fill_normal(128, seed, 42, mean=1.0, std=0.1),
                X=lb.fill_normal(H, seed, 43, std=1.5), w_post=lb.fill_normal(H, seed, 44, std=0.02, dtype="bf16"),
                w_in=lb.fill_normal(H, seed, 45, std=0.02, dtype="bf16"))
    return mats, dev, host


def _run_layer(ctx, lb, dev, host, chained, H=5120, V=6144, I=17408, NIN=16384):
    d = {k: ctx.to_device(v) for k, v in host.items()}
    d_m, d_y, d_xn = ctx.alloc(I * 2), ctx.alloc(NIN * 4), ctx.alloc(H * 2)
    ops = [_op(dev["out"], d["mix"], d["X"], V, H, lb.X_F32_HEADNORM_SILU, lb.Y_F32_ACCUM, aux0=d["hw"], aux1=d["z"]),
           _op(dev["gu"], d["X"], d_m, H, 2 * I, lb.X_F32_RMSNORM, lb.Y_SWIGLU_F16, aux0=d["w_post"]),
           _op(dev["down"], d_m, d["X"], I, H, lb.X_F16, lb.Y_F32_ACCUM),
           _op(dev["in"], d["X"], d_y, H, NIN, lb.X_F32_RMSNORM, lb.Y_F32, aux0=d["w_in"], x_out=d_xn)]
    if chained:
        ctx.gemv_chain(ops)
    else:
        for o in ops:
            ctx.gemv_int4_fused(o["qweight"], o["scales"], o["qzeros"], o["x"], o["y"], o["K"], o["N"], o["x_mode"], o["y_mode"],
                                aux0=o["aux0"], aux1=o["aux1"], x_out=o["x_out"])
    out = dict(X=d["X"].download(np.float32, H), m=d_m.download(np.float16, I).astype(np.float32), y=d_y.download(np.float32, NIN),
               xn=d_xn.download(np.float16, H).astype(np.float32))
    assert ctx.device_status() == 0
    for b in list(d.values()) + [d_m, d_y, d_xn]:
        b.free()
    return out


def test_layer_chain_vs_separate_launches_and_oracle(ctx, lb, oracle):
    H, V, I, NIN = 5120, 6144, 17408, 16384
    mats, dev, host = _layer_case(ctx, lb, 50)
    one = _run_layer(ctx, lb, dev, host, chained=False)
    ch = _run_layer(ctx, lb, dev, host, chained=True)
    ch2 = _run_layer(ctx, lb, dev, host, chained=True)
    ctx.set_chain_mailbox(False)                             # a grid barrier between every pair of entries instead of the tagged hand-over
    ch3 = _run_layer(ctx, lb, dev, host, chained=True)
    ctx.set_chain_mailbox(True)
    for k in one:
        assert rel_err_max(ch[k], one[k]) <= 2e-3, k        # different K partitions: same values to rounding
        assert np.array_equal(ch[k], ch2[k]), k              # run to run: bit-identical
        assert np.array_equal(ch[k], ch3[k]), k              # the hand-over carries the same values as the buffers
    # the same four steps on the CPU
    hn = np.concatenate([oracle.rmsnorm(host["mix"][i:i + 128], host["hw"], one_plus_w=False)[0] for i in range(0, V, 128)])
    hn = hn * (host["z"] / (1 + np.exp(-host["z"])))
    qw, sc, qz, _ = mats["out"]
    X1 = host["X"] + oracle.gptq_gemv(qw, sc, qz, hn.astype(np.float16), V, H)[0]
    h1, _ = oracle.rmsnorm(X1, oracle.bf16_to_f32(host["w_post"]), one_plus_w=True)
    qw, sc, qz, _ = mats["gu"]
    gu = oracle.gptq_gemv(qw, sc, qz, h1.astype(np.float16), H, 2 * I)[0].reshape(2 * I // 128, 2, 64)
    m = oracle.swiglu(gu[:, 0, :].ravel(), gu[:, 1, :].ravel())
    assert rel_err_max(ch["m"], m) <= 3e-3
    qw, sc, qz, _ = mats["down"]
    X2 = X1 + oracle.gptq_gemv(qw, sc, qz, m.astype(np.float16), I, H)[0]
    assert rel_err_max(ch["X"], X2) <= 3e-3
    h2, _ = oracle.rmsnorm(X2, oracle.bf16_to_f32(host["w_in"]), one_plus_w=True)
    qw, sc, qz, _ = mats["in"]
    y = oracle.gptq_gemv(qw, sc, qz, h2.astype(np.float16), H, NIN)[0]
    assert rel_err_max(ch["y"], y) <= 3e-3
    assert rel_err_max(ch["xn"], h2) <= 3e-3
    for v in dev.values():
        for b in v:
            if b:
                b.free()


def test_chain_in_a_graph(ctx, lb):
    """captured once, replayed three times: each replay continues from the previous residual stream"""
    K, N = 5120, 5120
    qw, sc, qz, _ = gptq_case(K, N, seed=60)
    d = _dev(ctx, qw, sc, qz, K, N)
    x0 = lb.fill_normal(K, 60, 5, std=0.5)
    w = lb.fill_normal(K, 60, 6, std=0.02, dtype="bf16")
    d_w = ctx.to_device(w)
    res = []
    for graph in (False, True):
        d_a, d_b = ctx.to_device(x0), ctx.to_device(x0[::-1].copy())
        # a GEMV's x and y never overlap: a -> b, then b -> a
        ops = [_op(d, d_a, d_b, K, N, lb.X_F32_RMSNORM, lb.Y_F32_ACCUM, aux0=d_w),
               _op(d, d_b, d_a, K, N, lb.X_F32_RMSNORM, lb.Y_F32_ACCUM, aux0=d_w)]
        if graph:
            ctx.begin_capture()
            ctx.gemv_chain(ops)
            g = ctx.end_capture()
            for _ in range(3):
                g.launch()
            ctx.sync()
        else:
            for _ in range(3):
                ctx.gemv_chain(ops)
        res.append(np.concatenate([d_a.download(np.float32, K), d_b.download(np.float32, K)]))
        assert ctx.device_status() == 0
        d_a.free()
        d_b.free()
    assert np.all(np.isfinite(res[0])) and np.array_equal(res[0], res[1])
    for b in d + [d_w]:
        b.free()


def test_chain_rejects_what_it_cannot_run(ctx, lb):
    d = ctx.alloc(1 << 16)
    with pytest.raises(lb.LithosError) as e:      # 38144 columns: more than 256 on one SM
        ctx.gemv_chain([dict(packed=d, x=d, y=d, K=1024, N=38144 + 256 * 148, x_mode=lb.X_F16, y_mode=lb.Y_F32)])
    assert e.value.status == lb.LB_ERR_INVALID
    with pytest.raises(lb.LithosError):           # K not a multiple of the group size
        ctx.gemv_chain([dict(packed=d, x=d, y=d, K=1000, N=1024, x_mode=lb.X_F16, y_mode=lb.Y_F32)])
    with pytest.raises(lb.LithosError):           # no packed weights
        ctx.gemv_chain([dict(packed=None, x=d, y=d, K=1024, N=1024, x_mode=lb.X_F16, y_mode=lb.Y_F32)])
    assert ctx.gemv_chain_supports(5120, 34816, swiglu=True) and not ctx.gemv_chain_supports(5120, 2 * 37888 + 128)
    d.free()


def test_timeline_hook(ctx, lb):
    """lb_set_chain_timeline: per SM and entry one %globaltimer stamp and seven cycle-counter stamps, in order, and nothing
    written once it is off"""
    K, N = 1024, 8192
    qw, sc, qz, x = gptq_case(K, N, seed=70)
    d = _dev(ctx, qw, sc, qz, K, N)
    d_x, d_y = ctx.to_device(x), ctx.alloc(N * 4)
    n_sm = ctx.sm_count
    tl = ctx.alloc(n_sm * 32 * 8 * 8).zero()
    lb.lib().lb_set_chain_timeline(ctx.h, tl.ptr)
    ctx.gemv_chain([_op(d, d_x, d_y, K, N, lb.X_F16, lb.Y_F32)] * 2)   # the second entry does not read the first one's result: a grid barrier separates them
    ctx.sync()
    lb.lib().lb_set_chain_timeline(ctx.h, 0)
    t = tl.download(np.uint64, n_sm * 32 * 8).reshape(n_sm, 32, 8).astype(np.int64)
    assert (t[:, :2, :] > 0).all() and (t[:, 2:, :] == 0).all()
    cyc = t[:, :, 1:]                                        # the SM's cycle counter: ordered inside an entry and from entry 0 to entry 1
    assert (np.diff(cyc[:, 0, :], axis=1) >= 0).all() and (np.diff(cyc[:, 1, :], axis=1) >= 0).all()
    assert (cyc[:, 1, 0] >= cyc[:, 0, 6]).all()
    assert (t[:, 1, 0] >= t[:, 0, 0]).all()                  # %globaltimer: the one stamp that compares across SMs
    assert (cyc[:, 1, 1] > cyc[:, 1, 0]).all()               # entry 1 passed a grid barrier
    tl.zero()
    ctx.gemv_chain([_op(d, d_x, d_y, K, N, lb.X_F16, lb.Y_F32)])
    ctx.sync()
    assert not tl.download(np.uint64, n_sm * 32 * 8).any()
    for b in d + [d_x, d_y, tl]:
        if b:
            b.free()


def test_gemv_int4_reads_the_packed_copy_once_there_is_one(ctx, lb, oracle):
    """lb_gemv_int4 on a matrix that lb_gemv_pack has packed runs as a chain of one (bit-identical to lb_gemv_chain), and goes
    back to the reference-format kernel when the copy is freed"""
    K, N = 5120, 17408
    qw, sc, qz, x = gptq_case(K, N, seed=77)
    want, _ = oracle.gptq_gemv(qw, sc, qz, x, K, N)
    d = [ctx.to_device(qw), ctx.to_device(sc), ctx.to_device(qz)]
    d_x, y0, y1, y2, y3 = ctx.to_device(x), ctx.alloc(N * 4), ctx.alloc(N * 4), ctx.alloc(N * 4), ctx.alloc(N * 4)
    assert ctx.gemv_packed_copy(d[0], K, N) == 0
    ctx.gemv_int4(d[0], d[1], d[2], d_x, y0, K, N, lb.GEMV_Y_F32)
    packed = ctx.gemv_pack(d[0], d[1], d[2], K, N)
    assert ctx.gemv_packed_copy(d[0], K, N) == packed.ptr and ctx.gemv_packed_copy(d[0], K, N, swiglu=True) == 0
    ctx.gemv_int4(d[0], d[1], d[2], d_x, y1, K, N, lb.GEMV_Y_F32)
    ctx.gemv_chain([dict(packed=packed, x=d_x, y=y2, K=K, N=N, x_mode=lb.X_F16, y_mode=lb.Y_F32)])
    packed.free()
    assert ctx.gemv_packed_copy(d[0], K, N) == 0
    ctx.gemv_int4(d[0], d[1], d[2], d_x, y3, K, N, lb.GEMV_Y_F32)
    g = [b.download(np.float32, N) for b in (y0, y1, y2, y3)]
    assert ctx.device_status() == 0
    assert np.array_equal(g[1], g[2]) and np.array_equal(g[0], g[3])
    for got in g:
        assert rel_err_max(got, want) <= TOL
    for b in d + [d_x, y0, y1, y2, y3]:
        b.free()

