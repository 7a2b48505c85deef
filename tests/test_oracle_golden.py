"""CPU: the C oracle against the committed known-answer fixtures (tests/golden/kat_small.npz,
numpy float64 from the formulas).  Integer work is bit-exact; floating point is checked at
fp32-rounding level (the oracle is fp32, the fixture float64)."""
from pathlib import Path

import numpy as np
import pytest

G = np.load(Path(__file__).parent / "golden" / "kat_small.npz")


def test_nibble_order_by_hand(oracle):
    # nibble j of a packed word is weight k = 8*kp + j, low nibble first
    q = oracle.gptq_unpack(G["nibble_word"].reshape(1, 1), 8, 1)
    assert q[:, 0].tolist() == G["nibble_values"].tolist() == [0, 1, 2, 3, 4, 5, 6, 7]


def test_gptq_unpack_bit_exact(oracle):
    K, N = G["gptq_q"].shape
    assert np.array_equal(oracle.gptq_unpack(G["gptq_qweight"], K, N), G["gptq_q"])
    assert np.array_equal(oracle.gptq_unpack_zeros(G["gptq_qzeros"], K, N), G["gptq_z"])


def test_gptq_dequant_bit_exact(oracle):
    K, N = G["gptq_q"].shape
    # (q-z)*s has at most 16 significant bits: exact in fp32, so fma(q,s,-z*s) must equal it bit for bit
    w = oracle.gptq_dequant(G["gptq_qweight"], G["gptq_scales"], G["gptq_qzeros"], K, N)
    assert np.array_equal(w, G["gptq_w"])
    w8 = oracle.gptq_dequant(G["gptq_qweight"], G["gptq_scales"], None, K, N)
    assert np.array_equal(w8, G["gptq_w_sym"])


def test_gptq_gemv(oracle):
    K, N = G["gptq_q"].shape
    y32, y16 = oracle.gptq_gemv(G["gptq_qweight"], G["gptq_scales"], G["gptq_qzeros"], G["gptq_x"], K, N)
    ref = G["gptq_y"]
    assert np.max(np.abs(y32 - ref)) / np.max(np.abs(ref)) < 2e-6
    assert np.array_equal(y16, y32.astype(np.float16))
    y32s, _ = oracle.gptq_gemv(G["gptq_qweight"], G["gptq_scales"], None, G["gptq_x"], K, N)
    assert np.max(np.abs(y32s - G["gptq_y_sym"])) / np.max(np.abs(G["gptq_y_sym"])) < 2e-6
    # compat contract: fp32 x, zero-point 8, result added to y
    y0 = np.full(N, 0.5, dtype=np.float32)
    ya = oracle.gptq_gemv_f32_accum(G["gptq_qweight"], G["gptq_scales"], G["gptq_x"].astype(np.float32), y0, K, N)
    assert np.allclose(ya - 0.5, G["gptq_y_sym"], rtol=0, atol=2e-6 * np.max(np.abs(G["gptq_y_sym"])))


def test_deltanet_three_steps(oracle):
    state = G["dn_state0"].copy()
    HV, d = state.shape[0], state.shape[1]
    T, HK = G["dn_q"].shape[0], G["dn_q"].shape[1]
    for t in range(T):
        g, beta = oracle.decay_gate(G["dn_a"][t], G["dn_a_log"], G["dn_dt_bias"], G["dn_b"][t])
        assert np.allclose(g, G["dn_g"][t], rtol=2e-6) and np.allclose(beta, G["dn_beta"][t], rtol=2e-6)
        out = oracle.deltanet_step(state, oracle.bf16_to_f32(G["dn_q"][t]), oracle.bf16_to_f32(G["dn_k"][t]),
                                   oracle.bf16_to_f32(G["dn_v"][t]), None, g, beta, HV, HK, d)
        assert np.max(np.abs(out - G["dn_out"][t])) / np.max(np.abs(G["dn_out"][t])) < 1e-5
    fro = np.linalg.norm((state - G["dn_state_final"]).reshape(HV, -1), axis=1) / np.linalg.norm(
        G["dn_state_final"].reshape(HV, -1), axis=1)
    assert fro.max() < 1e-5


def test_deltanet_z_gate(oracle):
    state = G["dn_state0"].copy()
    s2 = state.copy()
    HV, d = state.shape[0], state.shape[1]
    q, k, v = (oracle.bf16_to_f32(G[n][0]) for n in ("dn_q", "dn_k", "dn_v"))
    g, beta = oracle.decay_gate(G["dn_a"][0], G["dn_a_log"], G["dn_dt_bias"], G["dn_b"][0])
    z = np.linspace(-3, 3, HV * d, dtype=np.float32).reshape(HV, d)
    o_plain = oracle.deltanet_step(state, q, k, v, None, g, beta, HV, 1, d)
    o_gate = oracle.deltanet_step(s2, q, k, v, z, g, beta, HV, 1, d)
    assert np.allclose(o_gate, o_plain * (z / (1 + np.exp(-z))), rtol=1e-5, atol=1e-7)


def test_attention_step(oracle):
    kc, vc = G["at_kc"].copy(), G["at_vc"].copy()
    pos = int(G["at_pos"][0])
    HQ, d = G["at_q"].shape
    HKV = G["at_k_new"].shape[0]
    f = oracle.bf16_to_f32
    out = oracle.attention_step(f(G["at_q"]), f(G["at_k_new"]), f(G["at_v_new"]), f(G["at_gate"]), f(G["at_q_norm_w"]),
                                f(G["at_k_norm_w"]), kc, vc, pos, HQ, HKV, d)
    assert np.max(np.abs(out - G["at_out"])) / np.max(np.abs(G["at_out"])) < 2e-5
    # the appended key row: bf16 of a value computed in fp32 vs float64 may differ by one ulp at most
    assert np.max(np.abs(kc[pos].astype(np.int32) - G["at_k_row"].astype(np.int32))) <= 1
    assert np.array_equal(vc[pos], G["at_v_new"])


def test_small_kernels(oracle):
    y, s = oracle.rmsnorm(G["rms_x"], G["rms_w"], res=G["rms_r"], one_plus_w=True)
    assert np.allclose(y, G["rms_y_1pw"], rtol=3e-6, atol=1e-7)
    assert np.array_equal(s, G["rms_x"] + G["rms_r"])
    y, _ = oracle.rmsnorm(G["rms_x"], G["rms_w"], res=G["rms_r"], one_plus_w=False)
    assert np.allclose(y, G["rms_y_w"], rtol=3e-6, atol=1e-8)
    assert np.allclose(oracle.l2norm(G["rms_x"]), G["l2_y"], rtol=3e-6, atol=1e-8)
    y, h = oracle.conv1d_step(G["conv_x"], G["conv_w"], G["conv_hist"])
    assert np.allclose(y, G["conv_y"], rtol=1e-5, atol=1e-6) and np.array_equal(h, G["conv_hist_new"])
    assert np.allclose(oracle.swiglu(G["sw_gate"], G["sw_up"]), G["sw_y"], rtol=1e-5, atol=1e-7)
    assert oracle.argmax(G["argmax_x"]) == int(G["argmax_idx"][0])  # first maximum wins
    assert np.array_equal(oracle.rope(G["rope_x"], 2, 256, 64, 0, 1e7), G["rope_x"])
    assert np.allclose(oracle.rope(G["rope_x"], 2, 256, 64, 3, 1e7), G["rope_y_pos3"], rtol=1e-5, atol=1e-6)


def test_strip_layout_is_a_permutation(oracle):
    """The strip-packed layout holds every packed word exactly once, for any SM count and for SwiGLU pairs, and its
    (scale, zero-point) words match the reference tensors."""
    from helpers import gptq_case
    K, N = 384, 256
    qw, sc, qz, _ = gptq_case(K, N, seed=3)
    tag = np.arange(K // 8 * N, dtype=np.uint32).reshape(K // 8, N)      # distinct words, so positions can be traced
    for n_sms, swiglu in ((148, False), (7, False), (5, True), (1, True)):
        out = oracle.pack_strips(tag, sc, qz, K, N, n_sms, swiglu).reshape(-1, 136)
        assert out.shape[0] == N // 8 * (K // 128)
        assert np.array_equal(np.sort(out[:, :128].ravel()), tag.ravel())
        # lane (g, t), word j of a record: row 16*group + t + 4*j of column 8*octet + g
        rec = out[0]
        col0 = int(rec[0]) % N
        assert int(rec[4 * 5 + 2]) == (0 * 16 + 1 + 4 * 2) * N + col0 + 1   # lane 5 = (g 1, t 1), j = 2, first K-group
        zeros = oracle.gptq_unpack_zeros(qz, K, N)
        assert np.array_equal((out[0, 128:] >> 16).astype(np.uint16).view(np.float16).astype(np.int64), zeros[0, col0:col0 + 8])
        assert np.array_equal((out[0, 128:] & 0xFFFF).astype(np.uint16), sc.view(np.uint16)[0, col0:col0 + 8])
