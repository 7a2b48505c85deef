"""CPU: the C oracle against answers computed from the REFERENCE'S OWN KERNEL TEXT.

tests/golden/ls_kat.npz was produced by tests/golden/make_ls_golden.py, which parses inference/*.ls with the
reference's bootstrap-py parser and evaluates the syntax trees statement by statement (float32).  The inputs are the
closed-form vectors of tests/golden/ls_inputs.py, regenerated here.  Tolerances are those of float32 arithmetic in a
different evaluation order (<= 2e-6 of the largest value; RoPE 2e-5 because the text multiplies position and
frequency in float32 while the oracle reduces the angle in double).

Also here: the oracle's twin of the seeded tensor generator gives the same bits as the product's lb_fill_*.
"""
import sys
from pathlib import Path

import numpy as np

sys.path.insert(0, str(Path(__file__).parent / "golden"))
import ls_inputs as I  # noqa: E402

G = np.load(Path(__file__).parent / "golden" / "ls_kat.npz")


def close(a, b, tol):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return float(np.max(np.abs(a - b))) <= tol * max(float(np.max(np.abs(b))), 1e-30)


def test_decay_gate_as_written_and_sigmoid(oracle):
    c = I.decay_gate_case()
    g, beta = oracle.decay_gate(c["a_proj"], c["a_log"], c["dt_bias"], c["b"], text_log2=True)
    assert close(g, G["decay_gate_text"], 2e-6)
    assert close(beta, G["gate_sigmoid"], 2e-6)
    # the primary contract (natural-log softplus) is the same formula with ln in place of lg: g_text = g ** (1/ln 2)
    g_nat, _ = oracle.decay_gate(c["a_proj"], c["a_log"], c["dt_bias"], c["b"])
    assert close(g_nat.astype(np.float64) ** (1.0 / np.log(2.0)), G["decay_gate_text"], 2e-5)


def test_deltanet_fused_two_tokens(oracle):
    c = I.deltanet_fused_case()
    state = c["state"].copy()
    for t in range(c["T"]):
        out = oracle.deltanet_step(state, c["q"][t], c["k"][t], c["v"][t], c["z"][t], c["decay"][t], c["beta"][t],
                                   c["HV"], c["HK"], c["d"])
        assert close(out, G["dnf_out"][t], 2e-6)
    assert close(state[:, [0, 5, 77, 127], :], G["dnf_state_rows"], 2e-6)
    assert np.allclose(state.astype(np.float64).sum(axis=(1, 2)), G["dnf_state_sum"], rtol=0, atol=1e-4)


def test_delta_update(oracle):
    c = I.delta_update_case()
    d = c["d"]
    state = c["state"].copy().reshape(1, d, d)
    zero_q = np.zeros((1, d), np.float32)
    oracle.deltanet_step(state, zero_q, c["k"].reshape(1, d), c["v"].reshape(1, d), None, np.array([c["decay"]], np.float32),
                         np.array([c["beta"]], np.float32), 1, 1, d)
    assert close(state[0], G["du_state"], 2e-6)


def test_conv1d_five_tokens(oracle):
    c = I.conv1d_case()
    hist = c["hist"].copy()
    for t in range(c["T"]):
        y, hist = oracle.conv1d_step(c["x"][t], c["w"], hist)
        assert close(y, G["conv_y"][t], 2e-6)
    assert np.array_equal(hist, G["conv_hist"])


def test_elementwise(oracle):
    c = I.elementwise_case()
    assert np.array_equal(c["a"] + c["b"], G["ew_residual_add"])
    assert np.array_equal(c["a"] * c["b"], G["ew_elemwise_mul"]) and np.array_equal(c["a"] * c["b"], G["ew_scale"])
    assert close(oracle.silu(c["a"]), G["ew_activate_silu"], 2e-6)
    # SwiGLU = activate_silu then elemwise_mul (kernels.ls:61-66)
    assert close(oracle.swiglu(c["a"], c["b"]), G["ew_activate_silu"] * c["b"], 2e-6)


def test_rope_interleaved_pairs(oracle):
    c = I.rope_case()
    assert close(oracle.rope(c["q"], 1, 256, 64, c["pos"], 1e7), G["rope_q"], 2e-5)
    assert close(oracle.rope(c["k"], 1, 256, 64, c["pos"], 1e7), G["rope_k"], 2e-5)
    assert np.array_equal(G["rope_q"][64:], c["q"][64:])       # dims past the rotary part pass through


def test_generator_twin_is_bit_identical(oracle, lb):
    n, seed = 4099, 20260413
    assert np.array_equal(oracle.fill_u32(n, seed, 7), lb.fill_u32(n, seed, 7))
    assert np.array_equal(oracle.fill_scales_f16(n, seed, 8).view(np.uint16), lb.fill_scales_f16(n, seed, 8).view(np.uint16))
    for dt in ("f32", "f16", "bf16"):
        a, b = oracle.fill_normal(n, seed, 9, 0.25, 0.02, dt), lb.fill_normal(n, seed, 9, 0.25, 0.02, dt)
        assert np.array_equal(a.view(np.uint8), b.view(np.uint8)), dt
    assert np.array_equal(oracle.fill_uniform(n, seed, 10, 0.0, 2.7), lb.fill_uniform(n, seed, 10, 0.0, 2.7))
    # and the synthetic model built from either side is the same model
    from lithos_b200 import model as M
    cfg = M.tiny()
    ocfg = oracle.ModelCfg(**{k: getattr(cfg, k) for k, _ in M.ModelCfg._fields_})
    for layer in (0, 3):
        for x, y in zip(oracle.synthetic_layer_slots(ocfg, 5, layer), M.synthetic_layer_slots(cfg, 5, layer)):
            assert (x is None) == (y is None)
            if x is not None:
                assert np.array_equal(x.view(np.uint8), y.view(np.uint8))
