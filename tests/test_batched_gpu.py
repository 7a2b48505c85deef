"""GPU: the batched int4 projection (lb_gemm_int4) through the C ABI against the CPU oracle.

Row b of Y must equal the oracle's batch-1 GEMV of row b of X:
  max|y - y_ref| / max|y_ref| <= 1e-3 per row (the GEMV tolerance; up to 32 tokens the kernel keeps q - z
  exact and accumulates in fp32, so the observed error is near 1e-6; from 33 tokens on it multiplies
  fp16-rounded weights, error near 2e-4), and must equal lb_gemv_int4 on the same row to the same tolerance.
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


def run_gemm(ctx, lb, d_qw, d_sc, d_qz, x, K, N, f32=True):
    B = x.shape[0]
    d_x = ctx.to_device(np.ascontiguousarray(x))
    d_y = ctx.to_device(np.full(B * N, np.nan, dtype=np.float32))  # every element must be overwritten
    ctx.gemm_int4(d_qw, d_sc, d_qz, d_x, d_y, K, N, B, lb.GEMV_Y_F32 if f32 else 0)
    y = d_y.download(np.float32 if f32 else np.float16, B * N).reshape(B, N)
    assert ctx.device_status() == 0
    d_x.free()
    d_y.free()
    return y


# (K, N): one column block, a ragged last block (N % 128 = 16), K splits over a cluster, a wide matrix
SHAPES = [(256, 128), (1024, 144), (5120, 640), (2176, 5120), (1024, 20480)]


@pytest.mark.parametrize("K,N", SHAPES)
@pytest.mark.parametrize("zeros", [True, False])
def test_rows_match_oracle(ctx, lb, K, N, zeros):
    qw, sc, qz, _ = gptq_case(K, N, seed=K + N, zeros=zeros)
    d_qw, d_sc = ctx.to_device(qw), ctx.to_device(sc)
    d_qz = ctx.to_device(qz) if zeros else None
    X = batch_x(K, 64, seed=N)
    ref = np.stack([orc.gptq_gemv(qw, sc, qz, X[b], K, N)[0] for b in range(8)])
    for B in (1, 3, 4, 8, 16, 17, 33, 64):
        y = run_gemm(ctx, lb, d_qw, d_sc, d_qz, X[:B], K, N)
        assert np.isfinite(y).all()
        nb = min(B, 8)
        for b in range(nb):
            assert rel_err_max(y[b], ref[b]) <= TOL, (B, b)
    y16 = run_gemm(ctx, lb, d_qw, d_sc, d_qz, X[:5], K, N, f32=False)
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
    # up to 32 tokens the arithmetic is the same in every kernel variant: bit-exact rows
    y32 = run_gemm(ctx, lb, d_qw, d_sc, d_qz, X[:32], K, N)
    for B in (1, 4, 9, 16, 31):
        y = run_gemm(ctx, lb, d_qw, d_sc, d_qz, X[:B], K, N)
        assert np.array_equal(y, y32[:B]), B
    # 33..64 tokens multiply fp16-rounded weights: same rows within the GEMV tolerance, and bit-exact among themselves
    y64 = run_gemm(ctx, lb, d_qw, d_sc, d_qz, X, K, N)
    for b in range(32):
        assert rel_err_max(y64[b], y32[b]) <= TOL
    y40 = run_gemm(ctx, lb, d_qw, d_sc, d_qz, X[:40], K, N)
    assert np.array_equal(y40, y64[:40])
    # a permutation of the tokens permutes the rows
    perm = np.random.default_rng(3).permutation(64)
    yp = run_gemm(ctx, lb, d_qw, d_sc, d_qz, X[perm], K, N)
    assert np.array_equal(yp, y64[perm])
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
    for K, N, B in ((100, 128, 4), (128, 24, 4), (128, 128, 0), (128, 128, 65)):
        with pytest.raises(lb_mod.LithosError):
            ctx.gemm_int4(d, d, None, d, d, K, N, B, lb.GEMV_Y_F32)
    with pytest.raises(lb_mod.LithosError):
        ctx.gemm_int4(d, d, None, d, d, 128, 128, 4, lb.GEMV_Y_ACCUM)
    d.free()
