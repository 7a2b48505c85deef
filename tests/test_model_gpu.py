"""GPU: the whole decode step (lb_model_*) against the CPU oracle on a small model of the same
structure (3 DeltaNet layers + 1 attention layer per period, head dims 128/256, GQA 3 and 6).

Checks: greedy tokens identical over 64 decode steps; logits within 2e-3 of max|logit| at every
step; recurrent state / caches within 2e-3 (Frobenius) after the run; the captured CUDA graph
replays the same tokens as launch-by-launch decoding; seeded (non-zero) DeltaNet state, conv
history and KV prefix are honoured."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
SEED = 1234


def build_pair(ctx, lb, oracle, cfg, seed=SEED):
    from lithos_b200 import model as M
    ocfg = oracle.ModelCfg(**{n: getattr(cfg, n) for n, _ in M.ModelCfg._fields_})
    slots = [M.synthetic_layer_slots(cfg, seed, l) for l in range(cfg.n_layers)]
    glob = M.synthetic_globals(cfg, seed)
    om = oracle.Model(ocfg, slots, glob)
    gm = M.Model(ctx, cfg)
    gm.fill_synthetic(seed)          # the library's own generator: must equal the Python-side tensors
    return gm, om


def rel(a, b):
    return float(np.max(np.abs(np.asarray(a, np.float64) - b)) / max(np.max(np.abs(b)), 1e-30))


def test_tiny_model_64_greedy_steps(ctx, lb, oracle):
    from lithos_b200 import model as M
    cfg = M.tiny(max_ctx=96)
    gm, om = build_pair(ctx, lb, oracle, cfg)
    tok_g = tok_o = 17
    worst = 0.0
    min_gap = 1e9
    for pos in range(64):
        nxt_o = om.decode(tok_o, pos)
        nxt_g = gm.decode(tok_g, pos)
        lo = om.logits().copy()
        worst = max(worst, rel(gm.logits(), lo))
        top2 = np.partition(lo, -2)[-2:]
        min_gap = min(min_gap, float(top2[1] - top2[0]) / float(np.max(np.abs(lo))))
        assert nxt_g == nxt_o, f"greedy tokens diverge at step {pos} (top-2 gap {min_gap:.2e}, logit err {worst:.2e})"
        tok_g, tok_o = nxt_g, nxt_o
    assert worst <= 2e-3
    # recurrent state and caches after 64 steps
    for l in range(cfg.n_layers):
        if cfg.is_fa(l):
            n = 64 * cfg.fa_kv_heads * 256
            kg = lb.bf16_to_f32(gm.get_state(l, 0, np.uint16, n))
            ko = lb.bf16_to_f32(om.k_cache(l).ravel()[:n])
            assert np.max(np.abs(kg - ko)) <= 2.0 ** -7 * np.max(np.abs(ko))
        else:
            n = cfg.dn_v_heads * 128 * 128
            sg = gm.get_state(l, 0, np.float32, n).reshape(cfg.dn_v_heads, -1).astype(np.float64)
            so = om.dn_state(l).reshape(cfg.dn_v_heads, -1).astype(np.float64)
            fro = np.linalg.norm(sg - so, axis=1) / np.linalg.norm(so, axis=1)
            assert fro.max() <= 2e-3
    gm.close()
    om.close()


def test_graph_replay_equals_eager(ctx, lb, oracle):
    from lithos_b200 import model as M
    cfg = M.tiny(max_ctx=64)
    gm = M.Model(ctx, cfg)
    gm.fill_synthetic(SEED)
    eager = []
    tok = 5
    for pos in range(24):
        tok = gm.decode(tok, pos)
        eager.append(tok)
    logits_eager = gm.logits()
    gm.reset_state()
    gm.capture()
    assert gm.step_kernels <= cfg.n_layers + 4        # embed, persistent chains broken only by the attention kernel, LM head, arg-max
    gm.set_input(5, 0)
    replayed = []
    for pos in range(24):
        gm.replay(1)
        replayed.append(gm.read_next())
    assert replayed == eager
    assert np.array_equal(gm.logits(), logits_eager)   # ordered reductions: bit-identical
    # the whole chain without host round trips gives the same final token
    gm.reset_state()
    gm.set_input(5, 0)
    gm.replay(24)
    assert gm.read_next() == eager[-1]
    gm.close()


def test_seeded_state_is_used(ctx, lb, oracle):
    """non-zero DeltaNet state, conv history and a KV prefix seeded on both sides, then 8 steps from pos 40"""
    from lithos_b200 import model as M
    cfg = M.tiny(max_ctx=64)
    gm, om = build_pair(ctx, lb, oracle, cfg, seed=77)
    P0 = 40
    for l in range(cfg.n_layers):
        if cfg.is_fa(l):
            n = P0 * cfg.fa_kv_heads * 256
            k = lb.fill_normal(n, 9, 1000 + l, dtype="bf16")
            v = lb.fill_normal(n, 9, 2000 + l, dtype="bf16")
            om.k_cache(l).ravel()[:n] = k
            om.v_cache(l).ravel()[:n] = v
            gm.set_state(l, 0, k)
            gm.set_state(l, 1, v)
        else:
            s = lb.fill_normal(cfg.dn_v_heads * 128 * 128, 9, 3000 + l, std=0.02)
            hist = lb.fill_normal(3 * cfg.conv_channels, 9, 4000 + l).reshape(3, cfg.conv_channels)
            om.dn_state(l)[...] = s.reshape(om.dn_state(l).shape)
            om.conv_hist(l)[...] = hist
            gm.set_state(l, 0, s)
            ring = np.zeros((4, cfg.conv_channels), np.float32)
            for t in range(3):                      # hist[t] is the token at position P0-1-t
                ring[(P0 - 1 - t) & 3] = hist[t]
            gm.set_state(l, 1, ring)
    tok_g = tok_o = 99
    for pos in range(P0, P0 + 8):
        tok_o = om.decode(tok_o, pos)
        tok_g = gm.decode(tok_g, pos)
        assert rel(gm.logits(), om.logits()) <= 2e-3
        assert tok_g == tok_o
    gm.close()
    om.close()


def test_full_width_layers_chain_vs_separate_launches_vs_oracle(ctx, lb, oracle):
    """Four layers at the benchmark's widths (hidden 5120, SwiGLU 17408, 48/16 DeltaNet heads, 24/4
    attention heads; small vocabulary): here the projections between token mixers run as one
    persistent chain launch.  Tokens equal the oracle's and those of the one-launch-per-projection
    path over 12 steps; logits within 2e-3; the captured graph replays the same tokens."""
    from lithos_b200 import model as M
    full = M.qwen35_27b(max_ctx=48, n_layers=4)
    cfg = M.ModelCfg(**{**{n: getattr(full, n) for n, _ in M.ModelCfg._fields_}, "vocab": 4096})
    gm, om = build_pair(ctx, lb, oracle, cfg, seed=77)
    g1 = M.Model(ctx, cfg)
    g1.fill_synthetic(77)
    g1.set_chain(False)
    assert gm.ctx.gemv_chain_supports(cfg.hidden, 2 * cfg.inter, swiglu=True)
    tok = 5
    toks, worst = [], 0.0
    for pos in range(12):
        n_o = om.decode(tok, pos)
        n_c = gm.decode(tok, pos)
        n_1 = g1.decode(tok, pos)
        worst = max(worst, rel(gm.logits(), om.logits()), rel(g1.logits(), om.logits()))
        assert n_c == n_o == n_1, f"step {pos}: chain {n_c}, separate launches {n_1}, oracle {n_o} (logit err {worst:.2e})"
        tok = n_o
        toks.append(tok)
    assert worst <= 2e-3
    assert gm.step_kernels < g1.step_kernels        # 4 layers: 4 mixers + chains, against 5 launches per layer
    # graph replay from the start on a fresh model: same tokens
    g2 = M.Model(ctx, cfg)
    g2.fill_synthetic(77)
    g2.capture()
    g2.set_input(5, 0)
    rep = []
    for _ in range(12):
        g2.replay(1)
        rep.append(g2.read_next())
    assert rep == toks
    for m in (gm, g1, g2):
        m.close()
    om.close()


def test_checkpoint_and_rollback(ctx, lb, oracle):
    """decode ahead from a checkpoint, roll back, decode again: the same tokens and bit-identical logits; the rolled-back
    run also equals a run that never speculated (the KV rows written while speculating are rewritten, never read)"""
    from lithos_b200 import model as M
    import lithos_b200 as lb_mod
    cfg = M.tiny(max_ctx=64)
    gm = M.Model(ctx, cfg)
    gm.fill_synthetic(SEED)
    with pytest.raises(lb_mod.LithosError):
        gm.rollback()                      # nothing to roll back to yet
    tok = 7
    for pos in range(10):
        tok = gm.decode(tok, pos)
    gm.checkpoint()
    t0 = tok
    first = []
    for pos in range(10, 18):              # speculate 8 tokens
        tok = gm.decode(tok, pos)
        first.append(tok)
    logits_first = gm.logits()
    # a different continuation from the same point, to dirty the state and the KV rows 10..17
    tok = (t0 + 1) % cfg.vocab
    for pos in range(10, 18):
        tok = gm.decode(tok, pos)
    gm.rollback()
    tok, second = t0, []
    for pos in range(10, 18):
        tok = gm.decode(tok, pos)
        second.append(tok)
    assert second == first
    assert np.array_equal(gm.logits(), logits_first)
    # the checkpoint survives a rollback: roll back once more
    gm.rollback()
    tok, third = t0, []
    for pos in range(10, 18):
        tok = gm.decode(tok, pos)
        third.append(tok)
    assert third == first
    gm.close()


def test_weights_loaded_from_a_weight_index_file(ctx, lb, oracle, tmp_path):
    """lb_save_weights -> weight_index.bin + shard -> lb_load_weights: the same tokens and bit-identical logits as the
    model loaded from the host tensors directly"""
    from lithos_b200 import model as M, weights as W
    cfg = M.tiny(max_ctx=32)
    slots = [M.synthetic_layer_slots(cfg, 11, l) for l in range(cfg.n_layers)]
    glob = M.synthetic_globals(cfg, 11)
    W.save_weights(tmp_path, cfg, slots, glob)
    a, b = M.Model(ctx, cfg), M.Model(ctx, cfg)
    W.load_weights(a, tmp_path)
    for l in range(cfg.n_layers):
        b.load_layer(l, slots[l])
    b.load_globals(glob)
    ta = tb = 9
    for pos in range(10):
        ta, tb = a.decode(ta, pos), b.decode(tb, pos)
        assert ta == tb
    assert np.array_equal(a.logits(), b.logits())
    with pytest.raises(lb.LithosError) as e:          # a second load into the same model is refused, nothing is overwritten
        W.load_weights(a, tmp_path)
    assert e.value.status == lb.LB_ERR_STATE
    c = M.Model(ctx, cfg)
    with pytest.raises(lb.LithosError) as e:
        W.load_weights(c, tmp_path / "nowhere")
    assert e.value.status == lb.LB_ERR_IO
    for m in (a, b, c):
        m.close()
