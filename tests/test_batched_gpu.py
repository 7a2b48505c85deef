"""GPU: the batched int4 projection (lb_gemm_int4) through the C ABI against the CPU oracle.

Row b of Y must equal the oracle's batch-1 GEMV of row b of X:
  max|y - y_ref| / max|y_ref| <= 1e-3 per row (the GEMV tolerance; the mma.sync kernels keep q - z exact up to
  32 tokens and accumulate in fp32, observed error near 1e-6; the tcgen05 kernel, 9..64 tokens, and the 64-token
  mma.sync variant multiply fp16-rounded weights, error near 2e-4), and must equal lb_gemv_int4 on the same row
  to the same tolerance.  Both paths are run at every size they accept (flags LB_GEMM_MMA_SYNC / LB_GEMM_TCGEN05).
  Results may not depend on the batch a row travels in (checked bit-exactly between batch sizes that use
  the same arithmetic).
"""
import numpy as np
import pytest

import oracle.oracle as orc
from helpers import gptq_case, rel_err_max

import lithos_b200 as lb_mod

pytestmark = pytest.mark.gpu
TOL = 1e-3


def batch_x(K, B, seed):
    return lb_mod.fill_normal(B * K, seed, 40, dtype="f16").reshape(B, K)


def run_gemm(ctx, lb, d_qw, d_sc, d_qz, x, K, N, f32=True, extra=0):
    B = x.shape[0]
    d_x = ctx.to_device(np.ascontiguousarray(x))
    d_y = ctx.to_device(np.full(B * N, np.nan, dtype=np.float32))  # every element must be overwritten
    ctx.gemm_int4(d_qw, d_sc, d_qz, d_x, d_y, K, N, B, (lb.GEMV_Y_F32 if f32 else 0) | extra)
    y = d_y.download(np.float32 if f32 else np.float16, B * N).reshape(B, N)
    assert ctx.device_status() == 0
    d_x.free()
    d_y.free()
    return y


# (K, N): one column block, a ragged last block (N % 128 = 16), K splits over a cluster, a wide matrix
SHAPES = [(256, 128), (1024, 144), (5120, 640), (2176, 5120), (1024, 20480)]


@pytest.mark.parametrize("K,N", SHAPES)
@pytest.mark.parametrize("zeros", [True, False])
@pytest.mark.parametrize("path", ["tcgen05", "mma_sync"])
def test_rows_match_oracle(ctx, lb, K, N, zeros, path):
    force = lb.GEMM_MMA_SYNC if path == "mma_sync" else lb.GEMM_TCGEN05
    qw, sc, qz, _ = gptq_case(K, N, seed=K + N, zeros=zeros)
    d_qw, d_sc = ctx.to_device(qw), ctx.to_device(sc)
    d_qz = ctx.to_device(qz) if zeros else None
    X = batch_x(K, 256, seed=N)
    ref = np.stack([orc.gptq_gemv(qw, sc, qz, X[b], K, N)[0] for b in range(8)])
    for B in (1, 3, 4, 8, 16, 17, 33, 64) + ((100, 128, 129, 200, 256) if path == "tcgen05" else ()):  # more than 64 tokens: tcgen05 only
        extra = force if B > 8 else 0  # up to 8 tokens there is only the mma.sync kernel
        y = run_gemm(ctx, lb, d_qw, d_sc, d_qz, X[:B], K, N, extra=extra)
        assert np.isfinite(y).all()
        nb = min(B, 8)
        for b in range(nb):
            assert rel_err_max(y[b], ref[b]) <= TOL, (B, b)
        if B > 64:  # the last row and one in the upper half of the batch (other columns of tensor memory)
            for b in (B - 1, B // 2 + 3):
                assert rel_err_max(y[b], orc.gptq_gemv(qw, sc, qz, X[b], K, N)[0]) <= TOL, (B, b)
    y16 = run_gemm(ctx, lb, d_qw, d_sc, d_qz, X[:12], K, N, f32=False, extra=force)
    for b in range(5):
        assert rel_err_max(y16[b], ref[b].astype(np.float16)) <= 2e-3  # + one fp16 rounding of the result
    for d in (d_qw, d_sc, d_qz):
        if d:
            d.free()


def test_rows_do_not_depend_on_the_batch(ctx, lb):
    K, N = 2048, 4096
    qw, sc, qz, _ = gptq_case(K, N, seed=77)
    d_qw, d_sc, d_qz = ctx.to_device(qw), ctx.to_device(sc), ctx.to_device(qz)
    X = batch_x(K, 64, seed=5)
    # mma.sync kernels, up to 32 tokens: the same exact-integer arithmetic in every variant, bit-exact rows
    y32 = run_gemm(ctx, lb, d_qw, d_sc, d_qz, X[:32], K, N, extra=lb.GEMM_MMA_SYNC)
    for B in (1, 4, 9, 16, 31):
        y = run_gemm(ctx, lb, d_qw, d_sc, d_qz, X[:B], K, N, extra=lb.GEMM_MMA_SYNC)
        assert np.array_equal(y, y32[:B]), B
    # the tensor-core kernel (and the 64-token mma.sync variant) multiply fp16-rounded weights: same rows within the
    # GEMV tolerance; a row does not depend on how many tokens travel with it or where it sits in the batch
    y64 = run_gemm(ctx, lb, d_qw, d_sc, d_qz, X, K, N)
    for b in range(32):
        assert rel_err_max(y64[b], y32[b]) <= TOL
    for B in (9, 16, 17, 40):
        y = run_gemm(ctx, lb, d_qw, d_sc, d_qz, X[:B], K, N, extra=lb.GEMM_TCGEN05)
        assert np.array_equal(y, y64[:B]), B
    perm = np.random.default_rng(3).permutation(64)
    yp = run_gemm(ctx, lb, d_qw, d_sc, d_qz, X[perm], K, N)
    assert np.array_equal(yp, y64[perm])
    y64m = run_gemm(ctx, lb, d_qw, d_sc, d_qz, X, K, N, extra=lb.GEMM_MMA_SYNC)
    for b in range(64):
        assert rel_err_max(y64m[b], y64[b]) <= TOL
    for d in (d_qw, d_sc, d_qz):
        d.free()


def test_matches_the_batch_1_gemv(ctx, lb):
    K, N = 5120, 2048
    qw, sc, qz, _ = gptq_case(K, N, seed=9)
    d_qw, d_sc, d_qz = ctx.to_device(qw), ctx.to_device(sc), ctx.to_device(qz)
    X = batch_x(K, 16, seed=6)
    y = run_gemm(ctx, lb, d_qw, d_sc, d_qz, X, K, N)
    d_x, d_y = ctx.alloc(K * 2), ctx.alloc(N * 4)
    for b in range(16):
        d_x.upload(X[b])
        ctx.gemv_int4(d_qw, d_sc, d_qz, d_x, d_y, K, N, lb.GEMV_Y_F32)
        assert rel_err_max(y[b], d_y.download(np.float32, N)) <= TOL
    for d in (d_qw, d_sc, d_qz, d_x, d_y):
        d.free()


def test_runs_inside_a_graph(ctx, lb):
    K, N, B = 1024, 1024, 16
    qw, sc, qz, _ = gptq_case(K, N, seed=11)
    d_qw, d_sc, d_qz = ctx.to_device(qw), ctx.to_device(sc), ctx.to_device(qz)
    X = batch_x(K, B, seed=8)
    d_x, d_y = ctx.to_device(X), ctx.alloc(B * N * 4)
    ctx.gemm_int4(d_qw, d_sc, d_qz, d_x, d_y, K, N, B, lb.GEMV_Y_F32)
    want = d_y.download(np.float32, B * N)
    d_y.zero()
    ctx.begin_capture()
    ctx.gemm_int4(d_qw, d_sc, d_qz, d_x, d_y, K, N, B, lb.GEMV_Y_F32)
    g = ctx.end_capture()
    g.launch()
    ctx.sync()
    assert np.array_equal(d_y.download(np.float32, B * N), want)
    g.destroy()
    for d in (d_qw, d_sc, d_qz, d_x, d_y):
        d.free()


def test_bad_arguments_are_rejected(ctx, lb):
    d = ctx.alloc(1 << 16)
    for K, N, B in ((100, 128, 4), (128, 24, 4), (128, 128, 0), (128, 128, 257)):
        with pytest.raises(lb_mod.LithosError):
            ctx.gemm_int4(d, d, None, d, d, K, N, B, lb.GEMV_Y_F32)
    with pytest.raises(lb_mod.LithosError):
        ctx.gemm_int4(d, d, None, d, d, 128, 128, 65, lb.GEMM_MMA_SYNC)   # the mma.sync kernels stop at 64 tokens
    for flags in (lb.GEMV_Y_ACCUM, lb.GEMM_TCGEN05, lb.GEMM_TCGEN05 | lb.GEMM_MMA_SYNC):  # tcgen05 needs 9 tokens or more
        with pytest.raises(lb_mod.LithosError):
            ctx.gemm_int4(d, d, None, d, d, 128, 128, 4, flags)
    d.free()
