"""GPU: BASELINE config 3 itself against the CPU oracle: 64 layers, hidden 5120, SwiGLU 17408, vocabulary 248 320,
recurrent state and 4096 KV rows seeded exactly as bench.py seeds them, 64 greedy decode steps from position 4096.

Every step the GPU is given the oracle's previous token (so one disagreement cannot hide the steps after it) and must
predict the oracle's next token.  The top-2 logit gap of every step is kept, so that a disagreement can be told from
a tie.  Logits must agree within 1e-2 of max|logit|: the contract rounds the input of every projection to fp16, so two
fp32 evaluations that differ only in summation order (1e-6 per projection) flip individual fp16 roundings (2^-11 each)
and drift apart over the 448 projections of a step.  The oracle against ITSELF with every projection summed in
descending instead of ascending k differs by 2.3e-3 .. 3.1e-3 at this size (tests/test_drift_cpu.py shows the effect on
four layers); GPU against oracle measures 2.0e-3 .. 5.5e-3.  The 2e-3 bound of the small-model tests is kept where it
is attainable (4 layers).  Needs about 20 GB of host memory and about a minute."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
SEED, CTX, STEPS = 20260413, 4096, 64


def test_config3_64_layers_64_greedy_steps_vs_oracle(ctx, lb, oracle):
    from lithos_b200 import model as M
    cfg = M.qwen35_27b(max_ctx=CTX + STEPS + 8)
    ocfg = oracle.ModelCfg(**{n: getattr(cfg, n) for n, _ in M.ModelCfg._fields_})
    gm = M.Model(ctx, cfg)
    gm.fill_synthetic(SEED)
    gm.seed_state(CTX, SEED)
    slots = [oracle.synthetic_layer_slots(ocfg, SEED, l) for l in range(cfg.n_layers)]
    om = oracle.Model(ocfg, slots, oracle.synthetic_globals(ocfg, SEED))
    oracle.seed_state(om, CTX, SEED)
    tok, worst, rows, wrong = 1, 0.0, [], []
    for i in range(STEPS):
        pos = CTX + i
        n_o = om.decode(tok, pos)
        n_g = gm.decode(tok, pos)
        lo = om.logits()
        scale = float(np.max(np.abs(lo)))
        err = float(np.max(np.abs(gm.logits() - lo))) / scale
        top2 = np.partition(lo, -2)[-2:]
        gap = float(top2[1] - top2[0]) / scale
        rows.append((i, n_o, n_g, err, gap))
        worst = max(worst, err)
        if n_g != n_o:
            wrong.append(i)
        tok = n_o
    report = "\n".join(f"step {i:2d}: oracle {a:6d} gpu {b:6d} logit err {e:.2e} top-2 gap {g:.2e}" for i, a, b, e, g in rows)
    print(report)
    assert not wrong, f"greedy tokens differ at steps {wrong}\n{report}"
    assert worst <= 1e-2, f"logits differ by {worst:.2e} of max|logit|\n{report}"
    # the state after the run.  Layer 0 sees the same inputs on both sides (the embedding row): 2e-3 (Frobenius per head), the
    # bound of the stand-alone DeltaNet test.  Deeper layers inherit the drift of their inputs described above: 2e-2.
    for l, tol in ((0, 2e-3), (30, 2e-2), (62, 2e-2)):
        n = cfg.dn_v_heads * 128 * 128
        sg = gm.get_state(l, 0, np.float32, n).reshape(cfg.dn_v_heads, -1).astype(np.float64)
        so = om.dn_state(l).reshape(cfg.dn_v_heads, -1).astype(np.float64)
        assert (np.linalg.norm(sg - so, axis=1) / np.linalg.norm(so, axis=1)).max() <= tol, l
    for l in (3, 63):
        n, off = STEPS * cfg.fa_kv_heads * 256, CTX * cfg.fa_kv_heads * 256
        kg = lb.bf16_to_f32(gm.get_state(l, 0, np.uint16, n, offset_bytes=off * 2))
        ko = lb.bf16_to_f32(om.k_cache(l).ravel()[off:off + n])
        assert np.max(np.abs(kg - ko)) <= 2.0 ** -4 * np.max(np.abs(ko))
    gm.close()
    om.close()
