"""Seeded inputs shared by the CPU and GPU tests (shapes and distributions of the
benchmark configurations; values come from the library's counter-based generator)."""
import numpy as np

import lithos_b200 as lb


def gptq_case(K, N, seed=1, zeros=True):
    """qweight [K/8,N] u32, scales [K/128,N] f16, qzeros [K/128,N/8] u32 (or None), x [K] f16"""
    qw = lb.fill_u32(K // 8 * N, seed, 1).reshape(K // 8, N)
    sc = lb.fill_scales_f16(K // 128 * N, seed, 2).reshape(K // 128, N)
    qz = lb.fill_u32(K // 128 * (N // 8), seed, 3).reshape(K // 128, N // 8) if zeros else None
    x = lb.fill_normal(K, seed, 4, dtype="f16")
    return qw, sc, qz, x


def rel_err_max(a, b):
    """max |a-b| / max |b| : the GEMV tolerance metric"""
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    return float(np.max(np.abs(a - b)) / max(np.max(np.abs(b)), 1e-30))


def deltanet_case(seed, HV=48, HK=16, d=128, steps=1):
    """Config-1 inputs: state N(0,0.02); q,k bf16 N(0,1) L2-normalised per head; v bf16 N(0,1);
    beta = sigmoid(N(0,1)); g from A_log~U(0,2.7), a~N(0,1), dt_bias~N(0,0.1)"""
    state = lb.fill_normal(HV * d * d, seed, 10, std=0.02).reshape(HV, d, d)
    q = lb.fill_normal(steps * HK * d, seed, 11).reshape(steps, HK, d)
    k = lb.fill_normal(steps * HK * d, seed, 12).reshape(steps, HK, d)
    q = q / np.sqrt((q * q).sum(-1, keepdims=True))
    k = k / np.sqrt((k * k).sum(-1, keepdims=True))
    v = lb.fill_normal(steps * HV * d, seed, 13).reshape(steps, HV, d)
    a = lb.fill_normal(steps * HV, seed, 14).reshape(steps, HV)
    b = lb.fill_normal(steps * HV, seed, 15).reshape(steps, HV)
    a_log = lb.fill_uniform(HV, seed, 16, 0.0, 2.7)
    dt_bias = lb.fill_normal(HV, seed, 17, std=0.1)
    q16, k16, v16 = lb.f32_to_bf16(q), lb.f32_to_bf16(k), lb.f32_to_bf16(v)
    return dict(state=state, q=q16, k=k16, v=v16, a=a, b=b, a_log=a_log, dt_bias=dt_bias)


def attention_case(seed, L, HQ=24, HKV=4, d=256):
    """Config-2 inputs: K,V bf16 [L,HKV,d] N(0,1) (row L-1 is overwritten by the decoded token);
    q bf16 [HQ,d], new k,v bf16 [HKV,d], norm weights 1+N(0,0.02) bf16, gate N(0,1) bf16"""
    kc = lb.fill_normal(L * HKV * d, seed, 20, dtype="bf16").reshape(L, HKV, d)
    vc = lb.fill_normal(L * HKV * d, seed, 21, dtype="bf16").reshape(L, HKV, d)
    q = lb.fill_normal(HQ * d, seed, 22, dtype="bf16").reshape(HQ, d)
    kn = lb.fill_normal(HKV * d, seed, 23, dtype="bf16").reshape(HKV, d)
    vn = lb.fill_normal(HKV * d, seed, 24, dtype="bf16").reshape(HKV, d)
    gate = lb.fill_normal(HQ * d, seed, 25, dtype="bf16").reshape(HQ, d)
    qw = lb.fill_normal(d, seed, 26, mean=1.0, std=0.02, dtype="bf16")
    kw = lb.fill_normal(d, seed, 27, mean=1.0, std=0.02, dtype="bf16")
    return dict(kc=kc, vc=vc, q=q, k_new=kn, v_new=vn, gate=gate, q_norm_w=qw, k_norm_w=kw)
