"""Generates tests/golden/kat_small.npz: small known-answer cases for every kernel on
the decode path, computed here in numpy float64 straight from the formulas (bit
operations for the int4 unpack), independently of both the C oracle and the CUDA
kernels.  Inputs are stored with the answers, so the fixture does not depend on any
random generator at test time.

    python tests/golden/make_golden.py

The reference project ships no golden vectors for these kernels; these cases pin
the restated maths (formulas cited in oracle/oracle.c) and the packing conventions.
"""
from pathlib import Path

import numpy as np

rs = np.random.RandomState(20260413)
out = {}


def bf16_round(a):
    u = np.asarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    return r, (r.astype(np.uint32) << 16).view(np.float32)


# ---- 1. GPTQ int4 ---------------------------------------------------------------
K, N = 256, 32
qw = rs.randint(0, 2**32, size=(K // 8, N), dtype=np.uint64).astype(np.uint32)
qz = rs.randint(0, 2**32, size=(K // 128, N // 8), dtype=np.uint64).astype(np.uint32)
sc = (np.abs(rs.randn(K // 128, N)) * 0.01 + 1e-3).astype(np.float16)
x = rs.randn(K).astype(np.float16)
k = np.arange(K)
q = (qw[k // 8, :] >> (4 * (k % 8))[:, None].astype(np.uint32)) & 0xF          # [K,N]
n = np.arange(N)
z = (qz[:, n // 8] >> (4 * (n % 8))[None, :].astype(np.uint32)) & 0xF          # [K/128,N]
W = (q.astype(np.float64) - z[k // 128, :].astype(np.float64)) * sc[k // 128, :].astype(np.float64)
W8 = (q.astype(np.float64) - 8.0) * sc[k // 128, :].astype(np.float64)
out.update(gptq_qweight=qw, gptq_qzeros=qz, gptq_scales=sc, gptq_x=x, gptq_q=q.astype(np.uint8),
           gptq_z=z.astype(np.uint8), gptq_w=W.astype(np.float32), gptq_w_sym=W8.astype(np.float32),
           gptq_y=(W.T @ x.astype(np.float64)), gptq_y_sym=(W8.T @ x.astype(np.float64)))
# the packing convention, by hand: nibble j of a word is weight k = 8*kp + j
out["nibble_word"] = np.array([0x76543210], dtype=np.uint32)
out["nibble_values"] = np.arange(8, dtype=np.uint8)

# ---- 2. gated DeltaNet, 3 steps --------------------------------------------------
HV, HK, d, T = 3, 1, 128, 3
S = (rs.randn(HV, d, d) * 0.02)
S0 = S.astype(np.float32).copy()
qs = rs.randn(T, HK, d); ks = rs.randn(T, HK, d)
qs /= np.linalg.norm(qs, axis=-1, keepdims=True); ks /= np.linalg.norm(ks, axis=-1, keepdims=True)
q_bits, q_f = bf16_round(qs); k_bits, k_f = bf16_round(ks)
v_bits, v_f = bf16_round(rs.randn(T, HV, d))
a = rs.randn(T, HV).astype(np.float32); b = rs.randn(T, HV).astype(np.float32)
a_log = rs.uniform(0, 2.7, HV).astype(np.float32); dt_bias = (rs.randn(HV) * 0.1).astype(np.float32)
g = np.exp(-np.exp(a_log.astype(np.float64)) * np.log1p(np.exp(a.astype(np.float64) + dt_bias)))
beta = 1.0 / (1.0 + np.exp(-b.astype(np.float64)))
S = S0.astype(np.float64)
outs = np.zeros((T, HV, d))
for t in range(T):
    for h in range(HV):
        kh = h // (HV // HK)
        kk, qq = k_f[t, kh].astype(np.float64), q_f[t, kh].astype(np.float64)
        r = kk @ S[h]                                   # S^T k (old, un-decayed state)
        delta = beta[t, h] * (v_f[t, h].astype(np.float64) - r)
        S[h] = g[t, h] * S[h] + np.outer(kk, delta)
        outs[t, h] = qq @ S[h]
out.update(dn_state0=S0, dn_q=q_bits, dn_k=k_bits, dn_v=v_bits, dn_a=a, dn_b=b, dn_a_log=a_log, dn_dt_bias=dt_bias,
           dn_g=g, dn_beta=beta, dn_state_final=S.astype(np.float32), dn_out=outs)

# ---- 3. GQA decode attention (norm + RoPE + append + softmax + gate) ---------------
L, HQ, HKV, D, ROT, THETA, EPS = 40, 6, 2, 256, 64, 1e7, 1e-6
pos = L - 1
kc_bits, kc = bf16_round(rs.randn(L, HKV, D)); vc_bits, vc = bf16_round(rs.randn(L, HKV, D))
qr_bits, qr = bf16_round(rs.randn(HQ, D)); kn_bits, kn = bf16_round(rs.randn(HKV, D)); vn_bits, vn = bf16_round(rs.randn(HKV, D))
gt_bits, gt = bf16_round(rs.randn(HQ, D))
qw_bits, qwn = bf16_round(1 + 0.02 * rs.randn(D)); kw_bits, kwn = bf16_round(1 + 0.02 * rs.randn(D))


def norm_rope(v, w):
    v = v.astype(np.float64)
    v = v / np.sqrt((v * v).mean(-1, keepdims=True) + EPS) * w.astype(np.float64)
    i = np.arange(ROT // 2)
    ang = pos * np.exp2(-np.log2(THETA) * i / (ROT // 2))
    c, s = np.cos(ang), np.sin(ang)
    o = v.copy()
    o[..., 0:ROT:2] = v[..., 0:ROT:2] * c - v[..., 1:ROT:2] * s
    o[..., 1:ROT:2] = v[..., 0:ROT:2] * s + v[..., 1:ROT:2] * c
    return o


qn = norm_rope(qr, qwn)
knn_bits, knn = bf16_round(norm_rope(kn, kwn).astype(np.float32))
kc2, vc2 = kc.astype(np.float64).copy(), vc.astype(np.float64).copy()
kc2[pos], vc2[pos] = knn, vn
ao = np.zeros((HQ, D))
for h in range(HQ):
    kv = h * HKV // HQ
    s = (kc2[:, kv, :] @ qn[h]) / np.sqrt(D)
    p = np.exp(s - s.max()); p /= p.sum()
    ao[h] = (p @ vc2[:, kv, :]) / (1 + np.exp(-gt[h].astype(np.float64)))
out.update(at_kc=kc_bits, at_vc=vc_bits, at_q=qr_bits, at_k_new=kn_bits, at_v_new=vn_bits, at_gate=gt_bits,
           at_q_norm_w=qw_bits, at_k_norm_w=kw_bits, at_out=ao, at_k_row=knn_bits, at_pos=np.array([pos]))

# ---- 4. small kernels ------------------------------------------------------------------
D = 512
xv = rs.randn(D).astype(np.float32); rv = rs.randn(D).astype(np.float32); wv = (0.1 * rs.randn(D)).astype(np.float32)
sv = xv.astype(np.float64) + rv
out.update(rms_x=xv, rms_r=rv, rms_w=wv,
           rms_y_1pw=sv / np.sqrt((sv * sv).mean() + 1e-6) * (1 + wv.astype(np.float64)),
           rms_y_w=sv / np.sqrt((sv * sv).mean() + 1e-6) * wv.astype(np.float64),
           l2_y=xv.astype(np.float64) / np.sqrt((xv.astype(np.float64) ** 2).sum()))
C = 64
cx = rs.randn(C).astype(np.float32); cw = rs.randn(4, C).astype(np.float32); ch = rs.randn(3, C).astype(np.float32)
cy = cw[0].astype(np.float64) * cx + cw[1] * ch[0].astype(np.float64) + cw[2] * ch[1].astype(np.float64) + cw[3] * ch[2].astype(np.float64)
out.update(conv_x=cx, conv_w=cw, conv_hist=ch, conv_y=cy, conv_hist_new=np.stack([cx, ch[0], ch[1]]))
gg = rs.randn(D).astype(np.float32); uu = rs.randn(D).astype(np.float32)
out.update(sw_gate=gg, sw_up=uu, sw_y=gg.astype(np.float64) / (1 + np.exp(-gg.astype(np.float64))) * uu)
am = rs.randn(1000).astype(np.float32); am[[123, 777]] = am.max() + 1.0   # a tie: the first index must win
out.update(argmax_x=am, argmax_idx=np.array([123]))
# RoPE alone: pos = 0 is the identity; known rotation at pos = 3
rx = rs.randn(2, 256).astype(np.float32)
i = np.arange(32); ang = 3 * np.exp2(-np.log2(1e7) * i / 32)
ry = rx.astype(np.float64).copy()
ry[:, 0:64:2] = rx[:, 0:64:2] * np.cos(ang) - rx[:, 1:64:2] * np.sin(ang)
ry[:, 1:64:2] = rx[:, 0:64:2] * np.sin(ang) + rx[:, 1:64:2] * np.cos(ang)
out.update(rope_x=rx, rope_y_pos3=ry)

np.savez_compressed(Path(__file__).with_name("kat_small.npz"), **out)
print("wrote", Path(__file__).with_name("kat_small.npz"), sum(v.nbytes for v in out.values()), "bytes raw")
