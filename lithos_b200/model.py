"""Host-side mirror of the decode-step API (lb_model_* in include/lithos_b200.h)."""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import Context, LithosError, lib, fill_u32, fill_scales_f16, fill_normal, fill_uniform, LB_OK

WS_SLOTS, WG_SLOTS = 26, 3
# slot indices of the reference's per-layer weight table (src/launcher.s:92-141)
WS = dict(DN_QKV=0, DN_Z=3, DN_OUT=6, DN_PROJ_A=9, DN_PROJ_B=10, DN_A_LOG=11, DN_DT_BIAS=12, DN_CONV1D=13, DN_NORM=14,
          FA_Q=0, FA_K=3, FA_V=6, FA_O=9, FA_Q_NORM=12, FA_K_NORM=13, GATE=15, UP=18, DOWN=21, INPUT_NORM=24, POST_NORM=25)


class ModelCfg(C.Structure):
    _fields_ = [(n, C.c_int32) for n in (
        "n_layers", "hidden", "inter", "vocab", "dn_k_heads", "dn_v_heads", "dn_dim", "conv_taps",
        "fa_q_heads", "fa_kv_heads", "fa_dim", "rot_dims", "group", "fa_period", "max_ctx", "reserved")] + [
        ("eps", C.c_float), ("rope_theta", C.c_float)]

    def is_fa(self, layer: int) -> bool:
        return layer % self.fa_period == self.fa_period - 1

    @property
    def conv_channels(self) -> int:
        return (2 * self.dn_k_heads + self.dn_v_heads) * self.dn_dim


def qwen35_27b(max_ctx: int = 4224, n_layers: int = 64) -> ModelCfg:
    """models/families/qwen/qwen3.5/27b/config.json and src/launcher.s:62-72"""
    return ModelCfg(n_layers=n_layers, hidden=5120, inter=17408, vocab=248320, dn_k_heads=16, dn_v_heads=48, dn_dim=128,
                    conv_taps=4, fa_q_heads=24, fa_kv_heads=4, fa_dim=256, rot_dims=64, group=128, fa_period=4,
                    max_ctx=max_ctx, reserved=0, eps=1e-6, rope_theta=1e7)


def tiny(max_ctx: int = 128, n_layers: int = 4) -> ModelCfg:
    """same structure (3 DeltaNet + 1 attention per period, head dims 128/256, GQA 3 and 6), small widths"""
    return ModelCfg(n_layers=n_layers, hidden=1024, inter=2048, vocab=4096, dn_k_heads=2, dn_v_heads=6, dn_dim=128,
                    conv_taps=4, fa_q_heads=6, fa_kv_heads=1, fa_dim=256, rot_dims=64, group=128, fa_period=4,
                    max_ctx=max_ctx, reserved=0, eps=1e-6, rope_theta=1e7)


def synthetic_layer_slots(cfg: ModelCfg, seed: int, layer: int):
    """The host tensors lb_model_fill_synthetic generates for one layer (same streams), as a 26-slot list."""
    s = [None] * WS_SLOTS
    base = (layer + 1) * 100
    H, I = cfg.hidden, cfg.inter

    def q4(slot, K, N):
        s[slot] = fill_u32(K // 8 * N, seed, base + slot)
        s[slot + 1] = fill_scales_f16(K // 128 * N, seed, base + slot + 1)
        s[slot + 2] = fill_u32(K // 128 * (N // 8), seed, base + slot + 2)

    if not cfg.is_fa(layer):
        C_, V = cfg.conv_channels, cfg.dn_v_heads * 128
        q4(WS["DN_QKV"], H, C_)
        q4(WS["DN_Z"], H, V)
        q4(WS["DN_OUT"], V, H)
        s[WS["DN_PROJ_A"]] = fill_normal(cfg.dn_v_heads * H, seed, base + WS["DN_PROJ_A"], 0.0, 0.02, "bf16")
        s[WS["DN_PROJ_B"]] = fill_normal(cfg.dn_v_heads * H, seed, base + WS["DN_PROJ_B"], 0.0, 0.02, "bf16")
        s[WS["DN_A_LOG"]] = fill_uniform(cfg.dn_v_heads, seed, base + WS["DN_A_LOG"], 0.0, 2.7)
        s[WS["DN_DT_BIAS"]] = fill_normal(cfg.dn_v_heads, seed, base + WS["DN_DT_BIAS"], 0.0, 0.1, "bf16")
        s[WS["DN_CONV1D"]] = fill_normal(4 * C_, seed, base + WS["DN_CONV1D"], 0.0, 0.3, "bf16")
        s[WS["DN_NORM"]] = fill_normal(128, seed, base + WS["DN_NORM"], 1.0, 0.02, "f32")
    else:
        q4(WS["FA_Q"], H, 2 * cfg.fa_q_heads * 256)
        q4(WS["FA_K"], H, cfg.fa_kv_heads * 256)
        q4(WS["FA_V"], H, cfg.fa_kv_heads * 256)
        q4(WS["FA_O"], cfg.fa_q_heads * 256, H)
        s[WS["FA_Q_NORM"]] = fill_normal(256, seed, base + WS["FA_Q_NORM"], 1.0, 0.02, "bf16")
        s[WS["FA_K_NORM"]] = fill_normal(256, seed, base + WS["FA_K_NORM"], 1.0, 0.02, "bf16")
    q4(WS["GATE"], H, I)
    q4(WS["UP"], H, I)
    q4(WS["DOWN"], I, H)
    s[WS["INPUT_NORM"]] = fill_normal(H, seed, base + WS["INPUT_NORM"], 0.0, 0.02, "bf16")
    s[WS["POST_NORM"]] = fill_normal(H, seed, base + WS["POST_NORM"], 0.0, 0.02, "bf16")
    return s


def synthetic_globals(cfg: ModelCfg, seed: int):
    n = cfg.vocab * cfg.hidden
    return [fill_normal(n, seed, 1, 0.0, 0.02, "bf16"), fill_normal(n, seed, 2, 0.0, 0.02, "bf16"),
            fill_normal(cfg.hidden, seed, 3, 0.0, 0.02, "bf16")]


_sigs_done = False


def _sigs():
    global _sigs_done
    if _sigs_done:
        return
    L = lib()
    vp, i32, u64 = C.c_void_p, C.c_int, C.c_uint64
    P = C.POINTER
    L.lb_model_create.argtypes = [vp, P(ModelCfg), i32, i32, P(vp)]
    L.lb_model_destroy.argtypes = [vp]
    L.lb_model_destroy.restype = None
    L.lb_model_load_layer.argtypes = [vp, i32, P(vp)]
    L.lb_model_load_globals.argtypes = [vp, P(vp)]
    L.lb_model_fill_synthetic.argtypes = [vp, u64]
    L.lb_model_reset_state.argtypes = [vp]
    L.lb_model_checkpoint.argtypes = [vp]
    L.lb_model_rollback.argtypes = [vp]
    L.lb_model_state_ptr.argtypes = [vp, i32, i32, P(u64), P(C.c_size_t)]
    L.lb_model_logits_ptr.argtypes = [vp, P(u64)]
    L.lb_model_weight_bytes.argtypes = [vp]
    L.lb_model_weight_bytes.restype = u64
    L.lb_model_decode.argtypes = [vp, i32, i32, P(i32)]
    L.lb_model_capture.argtypes = [vp]
    L.lb_model_set_chain.argtypes = [vp, i32]
    L.lb_model_set_input.argtypes = [vp, i32, i32]
    L.lb_model_replay.argtypes = [vp, i32]
    L.lb_model_read_next.argtypes = [vp, P(i32)]
    L.lb_model_prefill.argtypes = [vp, P(i32), i32, i32, P(i32)]
    L.lb_model_set_sampling.argtypes = [vp, C.c_float, i32, u64]
    L.lb_model_generate.argtypes = [vp, P(i32), i32, i32, i32, P(i32), P(i32)]
    L.lb_model_step_kernels.argtypes = [vp]
    _sigs_done = True


class Model:
    """The decode step on one GPU (or one tensor-parallel shard)."""

    def __init__(self, ctx: Context, cfg: ModelCfg, tp_rank: int = 0, tp_size: int = 1):
        _sigs()
        self.ctx, self.cfg, self.tp_rank, self.tp_size = ctx, cfg, tp_rank, tp_size
        self.h = C.c_void_p(None)
        st = lib().lb_model_create(ctx.h, C.byref(cfg), tp_rank, tp_size, C.byref(self.h))
        if st != LB_OK:
            if self.h:
                lib().lb_model_destroy(self.h)
                self.h = None
            ctx._check(st)

    def close(self):
        if self.h:
            lib().lb_model_destroy(self.h)
            self.h = None

    def load_layer(self, layer: int, slots):
        arr = (C.c_void_p * WS_SLOTS)(*[(a.ctypes.data if a is not None else None) for a in slots])
        self.ctx._check(lib().lb_model_load_layer(self.h, layer, arr))

    def load_globals(self, g):
        arr = (C.c_void_p * WG_SLOTS)(*[a.ctypes.data for a in g])
        self.ctx._check(lib().lb_model_load_globals(self.h, arr))

    def fill_synthetic(self, seed: int):
        self.ctx._check(lib().lb_model_fill_synthetic(self.h, seed))

    def reset_state(self):
        self.ctx._check(lib().lb_model_reset_state(self.h))

    def checkpoint(self):
        """Snapshot the DeltaNet states and convolution histories (stream-ordered copies)."""
        self.ctx._check(lib().lb_model_checkpoint(self.h))

    def rollback(self):
        """Restore the last checkpoint; decoding continues from the checkpointed position."""
        self.ctx._check(lib().lb_model_rollback(self.h))

    def state_ptr(self, layer: int, which: int):
        p, n = C.c_uint64(0), C.c_size_t(0)
        self.ctx._check(lib().lb_model_state_ptr(self.h, layer, which, C.byref(p), C.byref(n)))
        return p.value, n.value

    def _xfer(self, ptr, arr, to_device):
        L = lib()
        if to_device:
            a = np.ascontiguousarray(arr)
            self.ctx._check(L.lb_memcpy_h2d(self.ctx.h, ptr, a.ctypes.data_as(C.c_void_p), a.nbytes))
        else:
            self.ctx._check(L.lb_memcpy_d2h(self.ctx.h, arr.ctypes.data_as(C.c_void_p), ptr, arr.nbytes))
        self.ctx.sync()

    def set_state(self, layer: int, which: int, arr: np.ndarray, offset_bytes: int = 0):
        p, n = self.state_ptr(layer, which)
        assert offset_bytes + arr.nbytes <= n
        self._xfer(p + offset_bytes, arr, True)

    def get_state(self, layer: int, which: int, dtype, count: int, offset_bytes: int = 0) -> np.ndarray:
        p, n = self.state_ptr(layer, which)
        out = np.empty(count, dtype=dtype)
        assert offset_bytes + out.nbytes <= n
        self._xfer(p + offset_bytes, out, False)
        return out

    def seed_state(self, ctx_len: int, seed: int):
        """Stand-in for a prompt of ctx_len tokens (the checkpoint and prompt of the reference's measurement are not
        distributable): ONE global seeded state, of which this shard takes its heads.  KV rows [0, ctx_len) bf16
        N(0,1) (streams 100000+l, 200000+l), DeltaNet state fp32 N(0,0.02) (300000+l), the three previous tokens'
        pre-convolution values fp32 N(0,1) (400000+l; row t = position ctx_len-1-t)."""
        cfg, R, T = self.cfg, self.tp_rank, self.tp_size
        HV, HK = cfg.dn_v_heads // T, cfg.dn_k_heads // T
        HKV = cfg.fa_kv_heads // T if cfg.fa_kv_heads >= T else 1
        kv0 = R * HKV if cfg.fa_kv_heads >= T else (R * cfg.fa_kv_heads) // T
        QKf, Cf = cfg.dn_k_heads * 128, cfg.conv_channels
        QK, V = HK * 128, HV * 128
        chan = np.concatenate([np.arange(R * QK, (R + 1) * QK), QKf + np.arange(R * QK, (R + 1) * QK),
                               2 * QKf + np.arange(R * V, (R + 1) * V)])
        for l in range(cfg.n_layers):
            if cfg.is_fa(l):
                n = ctx_len * cfg.fa_kv_heads * 256
                for which, stream in ((0, 100000 + l), (1, 200000 + l)):
                    rows = fill_normal(n, seed, stream, dtype="bf16").reshape(ctx_len, cfg.fa_kv_heads, 256)
                    self.set_state(l, which, np.ascontiguousarray(rows[:, kv0:kv0 + HKV]))
            else:
                st = fill_normal(cfg.dn_v_heads * 128 * 128, seed, 300000 + l, std=0.02).reshape(cfg.dn_v_heads, 128, 128)
                self.set_state(l, 0, np.ascontiguousarray(st[R * HV:(R + 1) * HV]))
                hist = fill_normal(3 * Cf, seed, 400000 + l).reshape(3, Cf)
                ring = np.zeros((4, chan.size), np.float32)
                for t in range(3):
                    ring[(ctx_len - 1 - t) & 3] = hist[t, chan]
                self.set_state(l, 1, ring)

    def logits(self) -> np.ndarray:
        p = C.c_uint64(0)
        self.ctx._check(lib().lb_model_logits_ptr(self.h, C.byref(p)))
        out = np.empty(self.cfg.vocab // self.tp_size, dtype=np.float32)  # this shard's vocabulary rows
        self._xfer(p.value, out, False)
        return out

    @property
    def weight_bytes(self) -> int:
        return lib().lb_model_weight_bytes(self.h)

    @property
    def step_kernels(self) -> int:
        return lib().lb_model_step_kernels(self.h)

    def decode(self, token: int, pos: int) -> int:
        nxt = C.c_int(0)
        self.ctx._check(lib().lb_model_decode(self.h, token, pos, C.byref(nxt)))
        return nxt.value

    def capture(self):
        self.ctx._check(lib().lb_model_capture(self.h))

    def set_chain(self, on: bool):
        """on (default): consecutive projections go out as one persistent launch; off: one launch each"""
        self.ctx._check(lib().lb_model_set_chain(self.h, 1 if on else 0))

    def set_input(self, token: int, pos: int):
        self.ctx._check(lib().lb_model_set_input(self.h, token, pos))

    def replay(self, n_steps: int = 1):
        self.ctx._check(lib().lb_model_replay(self.h, n_steps))

    def prefill(self, tokens, pos0: int = 0) -> int:
        """run the prompt through the model in chunks; returns the greedy token that follows it"""
        arr = (C.c_int * len(tokens))(*[int(t) for t in tokens])
        nxt = C.c_int(0)
        self.ctx._check(lib().lb_model_prefill(self.h, arr, len(tokens), pos0, C.byref(nxt)))
        return nxt.value

    def set_sampling(self, temperature: float, top_k: int, seed: int = 0):
        """top_k == 0: greedy; else temperature / top-k sampling, repeatable from (seed, position)"""
        self.ctx._check(lib().lb_model_set_sampling(self.h, temperature, top_k, seed))

    def generate(self, prompt, max_new: int, eos: int = -1):
        """the decode loop: prompt pass, then tokens until `eos`, max_new or a full context"""
        arr = (C.c_int * len(prompt))(*[int(t) for t in prompt])
        out, n = (C.c_int * max(max_new, 1))(), C.c_int(0)
        self.ctx._check(lib().lb_model_generate(self.h, arr, len(prompt), max_new, eos, out, C.byref(n)))
        return [out[i] for i in range(n.value)]

    def read_next(self) -> int:
        nxt = C.c_int(0)
        self.ctx._check(lib().lb_model_read_next(self.h, C.byref(nxt)))
        return nxt.value
