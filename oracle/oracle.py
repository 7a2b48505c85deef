"""ctypes wrapper of the CPU oracle (oracle/oracle.c) — TEST INFRASTRUCTURE.

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline legs may
import this module.  The product package never does.
"""
from __future__ import annotations

import ctypes as C
import subprocess
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
_LIB = _HERE / "liboracle.so"
REF_DIR = _HERE / "_ref"  # reference PTX assembled for sm_100a (built by the Makefile)


def reference_checkout():
    """The reference tree, when one is mounted: $LITHOS_REF, else a sibling `reference` directory of the repository's
    parent.  None on machines that only have the prebuilt files."""
    import os
    for cand in (os.environ.get("LITHOS_REF"), _HERE.parent.parent / "reference"):
        if cand and (Path(cand) / "minds").is_dir():
            return str(cand)
    return None


def build() -> None:
    targets, extra = ["liboracle.so"], []
    ref = reference_checkout()
    if ref:
        targets.append("ref")
        extra.append(f"LITHOS_REF={ref}")
    r = subprocess.run(["make", "-C", str(_HERE)] + targets + extra, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("oracle build failed:\n" + r.stdout[-2000:] + r.stderr[-2000:])


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not _LIB.exists():
            build()
        _lib = C.CDLL(str(_LIB))
        _lib.orc_num_threads.restype = C.c_int
        _lib.orc_argmax.restype = C.c_int
        _lib.orc_model_create.restype = C.c_void_p
        _lib.orc_model_decode.restype = C.c_int
        for n in ("orc_model_dn_state", "orc_model_conv_hist", "orc_model_k_cache", "orc_model_v_cache",
                  "orc_model_logits", "orc_model_residual"):
            getattr(_lib, n).restype = C.c_void_p
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def num_threads() -> int:
    return lib().orc_num_threads()


def set_sum_order(order: int) -> None:
    """0: every projection adds its K products in ascending k, 1: in descending k (both valid fp32 evaluations)"""
    lib().orc_set_sum_order(int(order))


def set_num_threads(n: int) -> None:
    lib().orc_set_num_threads(int(n))


# ---- seeded synthetic tensors: the twin of the product's lb_fill_* (same bits) ------------------
def _fill(n: int, seed: int, stream: int, kind: int, a: float, b: float, dtype) -> np.ndarray:
    out = np.empty(n, dtype=dtype)
    lib().orc_fill(_p(out), C.c_size_t(n), C.c_uint64(seed), C.c_uint64(stream), kind, C.c_float(a), C.c_float(b))
    return out


def fill_u32(n, seed, stream):
    return _fill(n, seed, stream, 0, 0.0, 0.0, np.uint32)


def fill_scales_f16(n, seed, stream):
    return _fill(n, seed, stream, 5, 0.0, 0.0, np.float16)


def fill_normal(n, seed, stream, mean=0.0, std=1.0, dtype="f32"):
    """dtype: 'f32' -> float32, 'f16' -> float16, 'bf16' -> uint16 holding bf16 bits"""
    kind, dt = {"f32": (1, np.float32), "f16": (2, np.float16), "bf16": (3, np.uint16)}[dtype]
    return _fill(n, seed, stream, kind, mean, std, dt)


def fill_uniform(n, seed, stream, lo, hi):
    return _fill(n, seed, stream, 4, lo, hi, np.float32)


def bf16_to_f32(a: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(a, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16(a: np.ndarray) -> np.ndarray:
    u = _f32(a).view(np.uint32).astype(np.uint64)
    r = (u + 0x7FFF + ((u >> 16) & 1)) >> 16
    return r.astype(np.uint16)


# ---- GPTQ -------------------------------------------------------------------
def gptq_unpack(qweight: np.ndarray, K: int, N: int) -> np.ndarray:
    out = np.empty((K, N), dtype=np.uint8)
    lib().orc_gptq_unpack(_p(qweight), K, N, _p(out))
    return out


def pack_strips(qweight, scales, qzeros, K: int, N: int, n_sms: int, swiglu: bool = False) -> np.ndarray:
    """The strip-packed weight layout of the persistent GEMV chain, restated with numpy (test infrastructure: the
    byte-exact target of lb_gemv_pack).  The reference keeps every matrix as qweight [K/8,N] / scales [K/128,N] /
    qzeros [K/128,N/8] (inference/gemv.ls:18-26); this layout holds the same numbers, reordered so that SM c owns
    the octets [start(c), start(c+1)), start(c) = floor(c * units / n_sms) * octets_per_unit, as one contiguous range:
    pair of octets by pair, K-group by K-group, per (octet, group) a record of 136 words: word 4*lane + j, lane =
    4*g + t, is the packed word of row 16*group + t + 4*j and column 8*octet + g; then 8 words (fp16 scale | fp16
    zero-point << 16).  With swiglu the input columns are interleaved 64-wide (gate, up) blocks and unit P is
    (gate octet, up octet) of output columns 8P..8P+7."""
    qw = np.asarray(qweight, dtype=np.uint32).reshape(K // 8, N)
    sc = np.asarray(scales).view(np.uint16).reshape(K // 128, N).astype(np.uint32)
    kg, no_total = K // 128, N // 8
    if qzeros is None:
        z = np.full((kg, N), 8, dtype=np.uint32)
    else:
        zw = np.asarray(qzeros, dtype=np.uint32).reshape(kg, N // 8)
        z = (zw[:, :, None] >> (4 * np.arange(8, dtype=np.uint32))[None, None, :]) & 0xF
        z = z.reshape(kg, N)
    zh = np.asarray(z, dtype=np.float16).view(np.uint16).astype(np.uint32)
    upo = 2 if swiglu else 1
    units = no_total // upo
    start = [(c * units // n_sms) * upo for c in range(n_sms + 1)]
    out = np.zeros(no_total * kg * 136, dtype=np.uint32)
    lane = np.arange(32)
    g_of, t_of = lane >> 2, lane & 3
    for c in range(n_sms):
        n0, no = start[c], start[c + 1] - start[c]
        for oi in range(no):
            O = n0 + oi
            if swiglu:
                P = O >> 1
                col0 = (P >> 3) * 128 + (O & 1) * 64 + (P & 7) * 8
            else:
                col0 = O * 8
            pair = oi >> 1
            recw = (2 if 2 * pair + 1 < no else 1) * 136
            for q in range(kg):
                dst = (n0 * kg + pair * kg * 2) * 136 + q * recw + (oi & 1) * 136
                rows = (16 * q + t_of[:, None] + 4 * np.arange(4)[None, :])          # [lane][j]
                out[dst:dst + 128] = qw[rows, (col0 + g_of)[:, None]].reshape(-1)
                out[dst + 128:dst + 136] = sc[q, col0:col0 + 8] | (zh[q, col0:col0 + 8] << 16)
    return out


def gptq_unpack_zeros(qzeros: np.ndarray, K: int, N: int, group: int = 128) -> np.ndarray:
    out = np.empty((K // group, N), dtype=np.uint8)
    lib().orc_gptq_unpack_zeros(_p(qzeros), K, N, group, _p(out))
    return out


def gptq_dequant(qweight, scales, qzeros, K: int, N: int, group: int = 128) -> np.ndarray:
    out = np.empty((K, N), dtype=np.float32)
    lib().orc_gptq_dequant(_p(qweight), _p(scales), _p(qzeros), K, N, group, _p(out))
    return out


def gptq_gemv(qweight, scales, qzeros, x_f16, K: int, N: int, group: int = 128):
    """returns (y_f32, y_f16)"""
    y32 = np.empty(N, dtype=np.float32)
    y16 = np.empty(N, dtype=np.float16)
    x = np.ascontiguousarray(x_f16, dtype=np.float16)
    lib().orc_gptq_gemv(_p(qweight), _p(scales), _p(qzeros), _p(x), _p(y32), _p(y16), K, N, group)
    return y32, y16


def gptq_gemv_f32_accum(qweight, scales, x_f32, y_f32, K: int, N: int) -> np.ndarray:
    y = _f32(y_f32).copy()
    lib().orc_gptq_gemv_f32_accum(_p(qweight), _p(scales), _p(_f32(x_f32)), _p(y), K, N)
    return y


def dense_bf16_gemv(w_bf16, x_f32, N: int, K: int) -> np.ndarray:
    y = np.empty(N, dtype=np.float32)
    lib().orc_dense_bf16_gemv(_p(w_bf16), _p(_f32(x_f32)), _p(y), N, K)
    return y


# ---- norms / elementwise -------------------------------------------------------
def rmsnorm(x, w, res=None, eps=1e-6, one_plus_w=True):
    x = _f32(x)
    y = np.empty_like(x)
    s = np.empty_like(x)
    lib().orc_rmsnorm(_p(x), _p(_f32(res)) if res is not None else None, _p(_f32(w)), _p(y), _p(s), x.size,
                      C.c_float(eps), 1 if one_plus_w else 0)
    return y, s


def l2norm(x):
    x = _f32(x)
    y = np.empty_like(x)
    lib().orc_l2norm(_p(x), _p(y), x.size)
    return y


def swiglu(gate, up, swap_operands=False):
    g, u = _f32(gate), _f32(up)
    y = np.empty_like(g)
    lib().orc_swiglu(_p(g), _p(u), _p(y), g.size, 1 if swap_operands else 0)
    return y


def conv1d_step(x, w, hist):
    """returns (y, new_hist); w [4,C], hist [3,C]"""
    x, w, h = _f32(x), _f32(w), _f32(hist).copy()
    y = np.empty_like(x)
    lib().orc_conv1d_step(_p(x), _p(w), _p(h), _p(y), x.size)
    return y, h


# ---- DeltaNet ------------------------------------------------------------------
def decay_gate(a, a_log, dt_bias, b, text_log2=False):
    """text_log2: softplus through log2 exactly as inference/decay_gate.ls:41-44 writes it (fixture pin only)"""
    a, a_log, dt_bias, b = _f32(a), _f32(a_log), _f32(dt_bias), _f32(b)
    g, beta = np.empty_like(a), np.empty_like(a)
    lib().orc_decay_gate_ex(_p(a), _p(a_log), _p(dt_bias), _p(b), _p(g), _p(beta), a.size, 1 if text_log2 else 0)
    return g, beta


def sigmoid(x):
    x = _f32(x)
    y = np.empty_like(x)
    lib().orc_sigmoid(_p(x), _p(y), x.size)
    return y


def silu(x):
    x = _f32(x)
    y = np.empty_like(x)
    lib().orc_silu(_p(x), _p(y), x.size)
    return y


def deltanet_step(state, q, k, v, z, g, beta, HV: int, HK: int, d: int = 128):
    """state is updated IN PLACE (must be a contiguous float32 array); returns out [HV,d]"""
    assert state.dtype == np.float32 and state.flags["C_CONTIGUOUS"]
    out = np.empty((HV, d), dtype=np.float32)
    lib().orc_deltanet_step(_p(state), _p(_f32(q)), _p(_f32(k)), _p(_f32(v)), _p(_f32(z)) if z is not None else None,
                            _p(_f32(g)), _p(_f32(beta)), _p(out), HV, HK, d)
    return out


# ---- attention ------------------------------------------------------------------
def rope(x, heads: int, d: int, rot_dims: int, pos: int, theta: float):
    x = _f32(x).copy()
    lib().orc_rope(_p(x), heads, d, rot_dims, pos, C.c_double(theta))
    return x


def rope_tables(n_pos: int, half: int, theta: float = 1e6):
    """cos / sin tables [n_pos, half] as the reference launcher precomputes them (src/launcher.s:3139-3148)"""
    c, s = np.empty((n_pos, half), np.float32), np.empty((n_pos, half), np.float32)
    lib().orc_rope_tables(_p(c), _p(s), n_pos, half, C.c_float(theta))
    return c, s


def rotate_half(x, heads: int, d: int, cos_t, sin_t, pos: int):
    """the launcher's half-split rotation of pairs (i, i + d/2) from the tables"""
    x = _f32(x).copy()
    lib().orc_rotate_half(_p(x), heads, d, _p(_f32(cos_t)), _p(_f32(sin_t)), pos)
    return x


def attention_decode(q, kc, vc, gate, L: int, HQ: int, HKV: int, d: int = 256):
    out = np.empty((HQ, d), dtype=np.float32)
    lib().orc_attention_decode(_p(_f32(q)), _p(kc), _p(vc), _p(_f32(gate)) if gate is not None else None, _p(out), L, HQ,
                               HKV, d)
    return out


def attention_step(q_raw, k_raw, v_new, gate, q_norm_w, k_norm_w, kc, vc, pos: int, HQ: int, HKV: int, d: int = 256,
                   rot_dims: int = 64, theta: float = 1e7, eps: float = 1e-6):
    """kc, vc (uint16 bf16 bits, [ctx,HKV,d]) get the new row appended IN PLACE; returns out [HQ,d]"""
    out = np.empty((HQ, d), dtype=np.float32)
    lib().orc_attention_step(_p(_f32(q_raw)), _p(_f32(k_raw)), _p(_f32(v_new)),
                             _p(_f32(gate)) if gate is not None else None, _p(_f32(q_norm_w)), _p(_f32(k_norm_w)),
                             _p(kc), _p(vc), _p(out), pos, HQ, HKV, d, rot_dims, C.c_double(theta), C.c_float(eps))
    return out


def embed_bf16(table, token: int, D: int):
    out = np.empty(D, dtype=np.float32)
    lib().orc_embed_bf16(_p(table), token, D, _p(out))
    return out


def argmax(x) -> int:
    x = _f32(x)
    return lib().orc_argmax(_p(x), x.size)


def topk_sample(x, temperature: float, top_k: int, u: float):
    """returns (token, top-k indices, their probabilities)"""
    x = _f32(x)
    idx, probs = np.zeros(64, np.int32), np.zeros(64, np.float32)
    lib().orc_topk_sample.restype = C.c_int
    tok = lib().orc_topk_sample(_p(x), x.size, C.c_float(temperature), int(top_k), C.c_float(u), _p(idx), _p(probs))
    k = max(1, min(64, int(top_k)))
    return tok, idx[:k], probs[:k]


# ---- whole model ------------------------------------------------------------------
class ModelCfg(C.Structure):
    _fields_ = [(n, C.c_int) for n in (
        "n_layers", "hidden", "inter", "vocab", "dn_k_heads", "dn_v_heads", "dn_dim", "conv_taps",
        "fa_q_heads", "fa_kv_heads", "fa_dim", "rot_dims", "group", "fa_period", "max_ctx", "reserved")] + [
        ("eps", C.c_float), ("rope_theta", C.c_float)]


WS_SLOTS, WG_SLOTS = 26, 3


class Model:
    """CPU model over a host weight table: layer_slots[l][slot] and globals[3] are numpy arrays."""

    def __init__(self, cfg: ModelCfg, layer_slots, globals_):
        self.cfg = cfg
        self._keep = (layer_slots, globals_)
        n = cfg.n_layers * WS_SLOTS
        self._slots = (C.c_void_p * n)()
        for l in range(cfg.n_layers):
            for s in range(WS_SLOTS):
                a = layer_slots[l][s]
                self._slots[l * WS_SLOTS + s] = a.ctypes.data if a is not None else None
        self._globals = (C.c_void_p * WG_SLOTS)(*[g.ctypes.data for g in globals_])
        self.h = C.c_void_p(lib().orc_model_create(C.byref(cfg), self._slots, self._globals))

    def _view(self, fn, layer, shape, dtype):
        p = getattr(lib(), fn)(self.h, layer)
        if not p:
            return None
        n = int(np.prod(shape))
        ct = {np.float32: C.c_float, np.uint16: C.c_uint16}[dtype]
        return np.ctypeslib.as_array(C.cast(p, C.POINTER(ct)), shape=(n,)).reshape(shape)

    def dn_state(self, layer):
        c = self.cfg
        return self._view("orc_model_dn_state", layer, (c.dn_v_heads, c.dn_dim, c.dn_dim), np.float32)

    def conv_hist(self, layer):
        c = self.cfg
        return self._view("orc_model_conv_hist", layer, (3, (2 * c.dn_k_heads + c.dn_v_heads) * c.dn_dim), np.float32)

    def k_cache(self, layer):
        c = self.cfg
        return self._view("orc_model_k_cache", layer, (c.max_ctx, c.fa_kv_heads, c.fa_dim), np.uint16)

    def v_cache(self, layer):
        c = self.cfg
        return self._view("orc_model_v_cache", layer, (c.max_ctx, c.fa_kv_heads, c.fa_dim), np.uint16)

    def logits(self):
        p = lib().orc_model_logits(self.h)
        return np.ctypeslib.as_array(C.cast(p, C.POINTER(C.c_float)), shape=(self.cfg.vocab,))

    def residual(self):
        p = lib().orc_model_residual(self.h)
        return np.ctypeslib.as_array(C.cast(p, C.POINTER(C.c_float)), shape=(self.cfg.hidden,))

    def decode(self, token: int, pos: int, n_layers_run: int = 0) -> int:
        return lib().orc_model_decode(self.h, token, pos, n_layers_run)

    def close(self):
        if self.h:
            lib().orc_model_destroy(self.h)
            self.h = None


# ---- the benchmark's synthetic model, built without the product library -------------------------
# Twins of lithos_b200.model.qwen35_27b / synthetic_layer_slots / synthetic_globals / Model.seed_state: the same
# streams of the same generator, so the CPU arm and the GPU arm of the benchmark decode the same model.
_WS = dict(DN_QKV=0, DN_Z=3, DN_OUT=6, DN_PROJ_A=9, DN_PROJ_B=10, DN_A_LOG=11, DN_DT_BIAS=12, DN_CONV1D=13, DN_NORM=14,
           FA_Q=0, FA_K=3, FA_V=6, FA_O=9, FA_Q_NORM=12, FA_K_NORM=13, GATE=15, UP=18, DOWN=21, INPUT_NORM=24, POST_NORM=25)


def qwen35_27b(max_ctx: int = 4224, n_layers: int = 64) -> ModelCfg:
    """models/families/qwen/qwen3.5/27b/config.json and src/launcher.s:62-72"""
    return ModelCfg(n_layers=n_layers, hidden=5120, inter=17408, vocab=248320, dn_k_heads=16, dn_v_heads=48, dn_dim=128,
                    conv_taps=4, fa_q_heads=24, fa_kv_heads=4, fa_dim=256, rot_dims=64, group=128, fa_period=4,
                    max_ctx=max_ctx, reserved=0, eps=1e-6, rope_theta=1e7)


def cfg_is_fa(cfg, layer: int) -> bool:
    return layer % cfg.fa_period == cfg.fa_period - 1


def synthetic_layer_slots(cfg, seed: int, layer: int):
    s = [None] * WS_SLOTS
    base = (layer + 1) * 100
    H, I = cfg.hidden, cfg.inter

    def q4(slot, K, N):
        s[slot] = fill_u32(K // 8 * N, seed, base + slot)
        s[slot + 1] = fill_scales_f16(K // 128 * N, seed, base + slot + 1)
        s[slot + 2] = fill_u32(K // 128 * (N // 8), seed, base + slot + 2)

    if not cfg_is_fa(cfg, layer):
        C_, V = (2 * cfg.dn_k_heads + cfg.dn_v_heads) * cfg.dn_dim, cfg.dn_v_heads * 128
        q4(_WS["DN_QKV"], H, C_)
        q4(_WS["DN_Z"], H, V)
        q4(_WS["DN_OUT"], V, H)
        s[_WS["DN_PROJ_A"]] = fill_normal(cfg.dn_v_heads * H, seed, base + _WS["DN_PROJ_A"], 0.0, 0.02, "bf16")
        s[_WS["DN_PROJ_B"]] = fill_normal(cfg.dn_v_heads * H, seed, base + _WS["DN_PROJ_B"], 0.0, 0.02, "bf16")
        s[_WS["DN_A_LOG"]] = fill_uniform(cfg.dn_v_heads, seed, base + _WS["DN_A_LOG"], 0.0, 2.7)
        s[_WS["DN_DT_BIAS"]] = fill_normal(cfg.dn_v_heads, seed, base + _WS["DN_DT_BIAS"], 0.0, 0.1, "bf16")
        s[_WS["DN_CONV1D"]] = fill_normal(4 * C_, seed, base + _WS["DN_CONV1D"], 0.0, 0.3, "bf16")
        s[_WS["DN_NORM"]] = fill_normal(128, seed, base + _WS["DN_NORM"], 1.0, 0.02, "f32")
    else:
        q4(_WS["FA_Q"], H, 2 * cfg.fa_q_heads * 256)
        q4(_WS["FA_K"], H, cfg.fa_kv_heads * 256)
        q4(_WS["FA_V"], H, cfg.fa_kv_heads * 256)
        q4(_WS["FA_O"], cfg.fa_q_heads * 256, H)
        s[_WS["FA_Q_NORM"]] = fill_normal(256, seed, base + _WS["FA_Q_NORM"], 1.0, 0.02, "bf16")
        s[_WS["FA_K_NORM"]] = fill_normal(256, seed, base + _WS["FA_K_NORM"], 1.0, 0.02, "bf16")
    q4(_WS["GATE"], H, I)
    q4(_WS["UP"], H, I)
    q4(_WS["DOWN"], I, H)
    s[_WS["INPUT_NORM"]] = fill_normal(H, seed, base + _WS["INPUT_NORM"], 0.0, 0.02, "bf16")
    s[_WS["POST_NORM"]] = fill_normal(H, seed, base + _WS["POST_NORM"], 0.0, 0.02, "bf16")
    return s


def synthetic_globals(cfg, seed: int):
    n = cfg.vocab * cfg.hidden
    return [fill_normal(n, seed, 1, 0.0, 0.02, "bf16"), fill_normal(n, seed, 2, 0.0, 0.02, "bf16"),
            fill_normal(cfg.hidden, seed, 3, 0.0, 0.02, "bf16")]


def seed_state(om: "Model", ctx_len: int, seed: int) -> None:
    """The benchmark's stand-in for a prompt of ctx_len tokens: KV rows [0, ctx_len) bf16 N(0,1) (streams 100000+l,
    200000+l), DeltaNet state fp32 N(0,0.02) (300000+l), the three previous tokens' pre-convolution values
    fp32 N(0,1) (400000+l; row t = position ctx_len-1-t).  Same tensors as lithos_b200.model.Model.seed_state."""
    cfg = om.cfg
    for l in range(cfg.n_layers):
        if cfg_is_fa(cfg, l):
            n = ctx_len * cfg.fa_kv_heads * cfg.fa_dim
            om.k_cache(l).ravel()[:n] = fill_normal(n, seed, 100000 + l, dtype="bf16")
            om.v_cache(l).ravel()[:n] = fill_normal(n, seed, 200000 + l, dtype="bf16")
        else:
            st = om.dn_state(l)
            st[...] = fill_normal(st.size, seed, 300000 + l, std=0.02).reshape(st.shape)
            h = om.conv_hist(l)
            h[...] = fill_normal(h.size, seed, 400000 + l).reshape(h.shape)
