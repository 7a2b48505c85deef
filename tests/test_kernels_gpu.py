"""GPU: gated DeltaNet, GQA decode attention and the small kernels through the C ABI
against the CPU oracle and the known-answer fixture.

Tolerances: DeltaNet state after 256 steps <= 2e-3 relative (Frobenius norm per head);
DeltaNet / attention outputs <= 2e-3 of max|out|; integer results (argmax, appended KV rows)
bit-exact."""
from pathlib import Path

import numpy as np
import pytest

from helpers import attention_case, deltanet_case, rel_err_max

pytestmark = pytest.mark.gpu
G = np.load(Path(__file__).parent / "golden" / "kat_small.npz")


def fro_rel(a, b):
    a = a.reshape(a.shape[0], -1).astype(np.float64)
    b = b.reshape(b.shape[0], -1).astype(np.float64)
    return float(np.max(np.linalg.norm(a - b, axis=1) / np.linalg.norm(b, axis=1)))


def test_deltanet_fixture(ctx, lb):
    T, HK = G["dn_q"].shape[:2]
    HV = G["dn_v"].shape[1]
    d_state = ctx.to_device(G["dn_state0"])
    d = {n: ctx.to_device(G["dn_" + n]) for n in ("q", "k", "v", "a", "b", "a_log", "dt_bias")}
    d_g, d_beta, d_out = ctx.alloc(T * HV * 4), ctx.alloc(T * HV * 4), ctx.alloc(T * HV * 128 * 4)
    # decay gate per step (a,b are [T,HV]; A_log and dt_bias are per head)
    a, b = G["dn_a"], G["dn_b"]
    for t in range(T):
        da, db = ctx.to_device(a[t]), ctx.to_device(b[t])
        dg, dbeta = ctx.alloc(HV * 4), ctx.alloc(HV * 4)
        ctx.decay_gate(da, d["a_log"], d["dt_bias"], db, dg, dbeta, HV)
        g = dg.download(np.float32, HV)
        beta = dbeta.download(np.float32, HV)
        assert np.allclose(g, G["dn_g"][t], rtol=1e-5) and np.allclose(beta, G["dn_beta"][t], rtol=1e-5)
    d_g.upload(G["dn_g"].astype(np.float32))
    d_beta.upload(G["dn_beta"].astype(np.float32))
    ctx.deltanet_step(d_state, d["q"], d["k"], d["v"], None, d_g, d_beta, d_out, HV, HK, n_steps=T)
    out = d_out.download(np.float32, T * HV * 128).reshape(T, HV, 128)
    assert rel_err_max(out, G["dn_out"]) <= 1e-4
    assert fro_rel(d_state.download(np.float32, HV * 128 * 128).reshape(HV, 128, 128), G["dn_state_final"]) <= 1e-4


def test_deltanet_256_steps_config1(ctx, lb, oracle):
    """BASELINE config 1: 48 value heads / 16 key heads, 256 consecutive steps, state drift <= 2e-3.
    Run both ways: 256 single-step launches, and one launch that keeps the state on chip."""
    HV, HK, T = 48, 16, 256
    c = deltanet_case(21, HV, HK, steps=T)
    g = np.empty((T, HV), np.float32)
    beta = np.empty((T, HV), np.float32)
    state = c["state"].copy()
    outs = np.empty((T, HV, 128), np.float32)
    qf, kf, vf = (oracle.bf16_to_f32(c[n]) for n in ("q", "k", "v"))
    for t in range(T):
        g[t], beta[t] = oracle.decay_gate(c["a"][t], c["a_log"], c["dt_bias"], c["b"][t])
        outs[t] = oracle.deltanet_step(state, qf[t], kf[t], vf[t], None, g[t], beta[t], HV, HK)
    d = {n: ctx.to_device(c[n]) for n in ("q", "k", "v")}
    d_g, d_beta = ctx.to_device(g), ctx.to_device(beta)
    d_out = ctx.alloc(T * HV * 128 * 4)
    # (a) one launch, state resident on chip for all 256 steps
    d_state = ctx.to_device(c["state"])
    ctx.deltanet_step(d_state, d["q"], d["k"], d["v"], None, d_g, d_beta, d_out, HV, HK, n_steps=T)
    s_a = d_state.download(np.float32, HV * 128 * 128).reshape(HV, 128, 128)
    o_a = d_out.download(np.float32, T * HV * 128).reshape(T, HV, 128)
    assert fro_rel(s_a, state) <= 2e-3
    assert rel_err_max(o_a, outs) <= 2e-3
    # (b) 256 launches of one step each; same arithmetic, so identical bits
    d_state.upload(c["state"])
    from lithos_b200 import DeviceBuffer
    step_q, step_v = HK * 128 * 2, HV * 128 * 2
    for t in range(T):
        views = []
        for name, stride in (("q", step_q), ("k", step_q), ("v", step_v)):
            v = DeviceBuffer.__new__(DeviceBuffer)
            v.ctx, v.ptr, v.nbytes = ctx, d[name].ptr + t * stride, stride
            views.append(v)
        vg, vb, vo = (DeviceBuffer.__new__(DeviceBuffer) for _ in range(3))
        vg.ctx, vg.ptr, vg.nbytes = ctx, d_g.ptr + t * HV * 4, HV * 4
        vb.ctx, vb.ptr, vb.nbytes = ctx, d_beta.ptr + t * HV * 4, HV * 4
        vo.ctx, vo.ptr, vo.nbytes = ctx, d_out.ptr + t * HV * 128 * 4, HV * 128 * 4
        ctx.deltanet_step(d_state, views[0], views[1], views[2], None, vg, vb, vo, HV, HK, n_steps=1)
    s_b = d_state.download(np.float32, HV * 128 * 128).reshape(HV, 128, 128)
    assert np.array_equal(s_a, s_b)
    assert np.array_equal(o_a, d_out.download(np.float32, T * HV * 128).reshape(T, HV, 128))


def test_deltanet_z_gate_and_f32_inputs(ctx, lb, oracle):
    HV, HK = 6, 2
    c = deltanet_case(22, HV, HK, steps=1)
    g, beta = oracle.decay_gate(c["a"][0], c["a_log"], c["dt_bias"], c["b"][0])
    z = lb.fill_normal(HV * 128, 22, 40).reshape(HV, 128)
    qf, kf, vf = (oracle.bf16_to_f32(c[n][0]) for n in ("q", "k", "v"))
    state = c["state"].copy()
    want = oracle.deltanet_step(state, qf, kf, vf, z, g, beta, HV, HK)
    d_state = ctx.to_device(c["state"])
    args = [ctx.to_device(a) for a in (qf, kf, vf, z, g, beta)]
    d_out = ctx.alloc(HV * 128 * 4)
    ctx.deltanet_step(d_state, args[0], args[1], args[2], args[3], args[4], args[5], d_out, HV, HK, in_is_f32=True)
    assert rel_err_max(d_out.download(np.float32, HV * 128), want.ravel()) <= 1e-4
    assert fro_rel(d_state.download(np.float32, HV * 128 * 128).reshape(HV, 128, 128), state) <= 1e-5


def run_attention(ctx, c, L, HQ, HKV, ctx_rows=None):
    rows = ctx_rows or L
    kc = np.zeros((rows, HKV, 256), np.uint16)
    vc = np.zeros((rows, HKV, 256), np.uint16)
    kc[:L], vc[:L] = c["kc"], c["vc"]
    d_kc, d_vc = ctx.to_device(kc), ctx.to_device(vc)
    d = {n: ctx.to_device(c[n]) for n in ("q", "k_new", "v_new", "gate", "q_norm_w", "k_norm_w")}
    d_out = ctx.alloc(HQ * 256 * 4)
    ctx.attention_decode(d["q"], d["k_new"], d["v_new"], d["gate"], d["q_norm_w"], d["k_norm_w"], d_kc, d_vc, d_out,
                         L - 1, HQ, HKV)
    out = d_out.download(np.float32, HQ * 256).reshape(HQ, 256)
    k_row = d_kc.download(np.uint16, HKV * 256, offset_bytes=(L - 1) * HKV * 256 * 2).reshape(HKV, 256)
    v_row = d_vc.download(np.uint16, HKV * 256, offset_bytes=(L - 1) * HKV * 256 * 2).reshape(HKV, 256)
    assert ctx.device_status() == 0
    for b in list(d.values()) + [d_kc, d_vc, d_out]:
        b.free()
    return out, k_row, v_row


def test_attention_fixture(ctx, lb):
    c = {n: G["at_" + n] for n in ("kc", "vc", "q", "k_new", "v_new", "gate", "q_norm_w", "k_norm_w")}
    L = int(G["at_pos"][0]) + 1
    HQ, HKV = c["q"].shape[0], c["k_new"].shape[0]
    out, k_row, v_row = run_attention(ctx, c, L, HQ, HKV)
    assert rel_err_max(out, G["at_out"]) <= 2e-3
    assert np.max(np.abs(k_row.astype(np.int32) - G["at_k_row"].astype(np.int32))) <= 1
    assert np.array_equal(v_row, G["at_v_new"])


@pytest.mark.parametrize("L", [1, 2, 77, 4096, 32768, 131072])
def test_attention_config2_vs_oracle(ctx, lb, oracle, L):
    """BASELINE config 2 (24 query / 4 KV heads, head_dim 256, RoPE on 64 dims, theta 1e7) at all three context
    lengths of the sweep (the oracle needs a few seconds at 131072); L = 1 and 2 are the empty / single-row cache
    edge cases."""
    HQ, HKV = 24, 4
    c = attention_case(31 + L, L, HQ, HKV)
    f = oracle.bf16_to_f32
    kc, vc = c["kc"].copy(), c["vc"].copy()
    want = oracle.attention_step(f(c["q"]), f(c["k_new"]), f(c["v_new"]), f(c["gate"]), f(c["q_norm_w"]), f(c["k_norm_w"]),
                                 kc, vc, L - 1, HQ, HKV)
    out, k_row, v_row = run_attention(ctx, c, L, HQ, HKV)
    assert rel_err_max(out, want) <= 2e-3
    # appended key row: one bf16 ulp of the row's largest value (rotation can cancel, so not ulp-of-element)
    kf, kw = f(k_row), f(kc[L - 1])
    assert np.max(np.abs(kf - kw)) <= 2.0 ** -7 * np.max(np.abs(kw))
    assert np.array_equal(v_row, vc[L - 1])


def test_attention_131072_properties(ctx, lb):
    """largest context of config 2: (1) run-to-run identical bits; (2) a cache whose V rows are all the
    same vector must return exactly that vector times the gate, whatever the scores are."""
    HQ, HKV, L = 24, 4, 131072
    c = attention_case(77, L, HQ, HKV)
    o1, _, _ = run_attention(ctx, c, L, HQ, HKV)
    o2, _, _ = run_attention(ctx, c, L, HQ, HKV)
    assert np.array_equal(o1, o2)
    vrow = c["v_new"]                                    # [HKV,256] bf16 bits
    c2 = dict(c)
    c2["vc"] = np.broadcast_to(vrow, (L, HKV, 256)).copy()
    o3, _, _ = run_attention(ctx, c2, L, HQ, HKV)
    v = (vrow.astype(np.uint32) << 16).view(np.float32)
    gate = (c["gate"].astype(np.uint32) << 16).view(np.float32)
    want = np.repeat(v, HQ // HKV, axis=0) / (1 + np.exp(-gate))
    assert rel_err_max(o3, want) <= 1e-4


def test_small_kernels(ctx, lb, oracle):
    D = 5120
    x = lb.fill_normal(2 * D, 41, 1, std=2.0)
    r = lb.fill_normal(2 * D, 41, 2)
    w = lb.fill_normal(D, 41, 3, std=0.05, dtype="bf16")
    d_x, d_r, d_w = ctx.to_device(x), ctx.to_device(r), ctx.to_device(w)
    d_y, d_s = ctx.alloc(2 * D * 4), ctx.alloc(2 * D * 4)
    ctx.rmsnorm(d_x, d_r, d_w, d_y, d_s, 2, D, one_plus_w=True)
    y = d_y.download(np.float32, 2 * D).reshape(2, D)
    for i in range(2):
        want, s = oracle.rmsnorm(x[i * D:(i + 1) * D], oracle.bf16_to_f32(w), res=r[i * D:(i + 1) * D])
        assert np.allclose(y[i], want, rtol=2e-5, atol=1e-6)
    assert np.array_equal(d_s.download(np.float32, 2 * D), x + r)
    # argmax: first maximum wins
    n = 248320
    lg = lb.fill_normal(n, 42, 1)
    lg[[5000, 200000]] = lg.max() + 1
    d_l, d_i = ctx.to_device(lg), ctx.alloc(16)
    ctx.argmax(d_l, n, d_i)
    assert int(d_i.download(np.int32, 1)[0]) == 5000 == oracle.argmax(lg)
    # embedding row gather, bf16 table
    V = 1000
    tab = lb.fill_normal(V * D, 43, 1, std=0.02, dtype="bf16")
    d_t, d_tok, d_e = ctx.to_device(tab), ctx.to_device(np.array([777], np.int32)), ctx.alloc(D * 4)
    ctx.embed(d_t, d_tok, d_e, D)
    assert np.array_equal(d_e.download(np.float32, D), oracle.embed_bf16(tab, 777, D))
    # dense bf16 matrix x vector (LM-head shape rows, fewer of them)
    N = 4096
    W = lb.fill_normal(N * D, 44, 1, std=0.02, dtype="bf16")
    xv = lb.fill_normal(D, 44, 2, dtype="f16")
    d_W, d_xv, d_o = ctx.to_device(W), ctx.to_device(xv), ctx.alloc(N * 4)
    ctx.dense_bf16_gemv(d_W, d_xv, d_o, N, D)
    want = oracle.dense_bf16_gemv(W, xv.astype(np.float32), N, D)
    assert rel_err_max(d_o.download(np.float32, N), want) <= 1e-5


def test_topk_sampling_vs_oracle(ctx, lb, oracle):
    """temperature + top-k sampling: the same candidates (ties by smaller index), probabilities within 1e-5, and the same
    token for every draw u that does not sit within 1e-5 of a step of the cumulative distribution"""
    n = 248320
    lg = lb.fill_normal(n, 91, 1, std=3.0)
    lg[[777, 200000]] = lg.max() + 0.5                         # a tie at the top: index 777 first
    d_l, d_tok = ctx.to_device(lg), ctx.alloc(16)
    d_p, d_i = ctx.alloc(64 * 4), ctx.alloc(64 * 4)
    seed = 20260413
    for k, T in ((1, 1.0), (8, 0.7), (50, 1.3), (64, 2.0)):
        for counter in range(6):
            u = float(lb.fill_uniform(counter + 1, seed, 7777, 0.0, 1.0)[counter])
            ctx.sample_topk(d_l, n, T, k, seed, counter, d_tok, d_p, d_i)
            tok = int(d_tok.download(np.int32, 1)[0])
            want, idx, probs = oracle.topk_sample(lg, T, k, u)
            assert np.array_equal(d_i.download(np.int32, 64)[:k], idx)
            gp = d_p.download(np.float32, 64)[:k]
            assert np.allclose(gp, probs, rtol=0, atol=1e-5)
            cdf = np.cumsum(probs.astype(np.float64))
            if np.min(np.abs(cdf - u)) > 1e-5:
                assert tok == want, (k, T, counter, u)
            assert tok in idx
        assert idx[0] == 777 and (k == 1 or idx[1] == 200000)


def test_generate_stops_at_eos_and_sampling_is_repeatable(ctx, lb):
    from lithos_b200 import model as M
    cfg = M.tiny(max_ctx=64)
    m = M.Model(ctx, cfg)
    m.fill_synthetic(1234)
    prompt = [5, 17, 300, 12]
    greedy = m.generate(prompt, 12)
    assert len(greedy) == 12
    m.reset_state()
    assert m.generate(prompt, 12, eos=greedy[4]) == greedy[:greedy.index(greedy[4]) + 1]   # stops right after the first end-of-sequence token
    # sampling: repeatable from (seed, position), different from greedy somewhere, different with another seed
    runs = []
    for seed in (7, 7, 8):
        m.reset_state()
        m.set_sampling(1.5, 40, seed)
        runs.append(m.generate(prompt, 24))
    assert runs[0] == runs[1] and runs[0] != runs[2] and runs[0] != greedy + [0] * 12
    m.set_sampling(1.0, 0, 0)
    m.reset_state()
    assert m.generate(prompt, 12) == greedy
    m.close()
