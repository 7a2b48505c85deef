"""Closed-form inputs shared by make_ls_golden.py (which evaluates the reference's .ls kernel text) and
tests/test_oracle_ls_pin.py (which runs the C oracle on the same inputs).  No random generator: element i
of vector `salt` is a pure integer hash, so the fixture only has to store the answers."""
import numpy as np


def hvec(n: int, salt: int, lo: float = -1.0, hi: float = 1.0) -> np.ndarray:
    """n float32 values in [lo, hi): a multiplicative hash of (salt, i), exact in every numpy version"""
    i = np.arange(n, dtype=np.uint64)
    with np.errstate(over="ignore"):   # arithmetic modulo 2^64 is the point
        h = (i + np.uint64(1)) * np.uint64(0x9E3779B97F4A7C15) + np.uint64((salt * 0xD1342543DE82EF95) & (2**64 - 1))
        h ^= h >> np.uint64(29)
        h *= np.uint64(0xBF58476D1CE4E5B9)
    h ^= h >> np.uint64(32)
    u = (h >> np.uint64(40)).astype(np.float64) / float(1 << 24)
    return (lo + (hi - lo) * u).astype(np.float32)


def unit_rows(a: np.ndarray) -> np.ndarray:
    """rows scaled to unit L2 norm (float32)"""
    a = a.astype(np.float64)
    return (a / np.sqrt((a * a).sum(-1, keepdims=True))).astype(np.float32)


# ---- the cases ---------------------------------------------------------------------------------
def decay_gate_case():
    n = 48
    return dict(a_proj=hvec(n, 1, -3, 3), a_log=hvec(n, 2, 0.0, 2.7), dt_bias=hvec(n, 3, -0.3, 0.3), b=hvec(n, 4, -3, 3))


def deltanet_fused_case():
    """2 key heads x 3 value heads, d = 128 (the kernel text hard-codes d = 128 and gqa = 3), two tokens"""
    HK, G, d, T = 2, 3, 128, 2
    HV = HK * G
    return dict(HK=HK, HV=HV, d=d, T=T,
                state=hvec(HV * d * d, 10, -0.05, 0.05).reshape(HV, d, d),
                q=unit_rows(hvec(T * HK * d, 11).reshape(T, HK, d)) * np.float32(0.08838834764831845),
                k=unit_rows(hvec(T * HK * d, 12).reshape(T, HK, d)),
                v=hvec(T * HV * d, 13).reshape(T, HV, d), z=hvec(T * HV * d, 14, -2, 2).reshape(T, HV, d),
                decay=hvec(T * HV, 15, 0.2, 1.0).reshape(T, HV), beta=hvec(T * HV, 16, 0.05, 0.95).reshape(T, HV))


def delta_update_case():
    d = 16
    return dict(d=d, state=hvec(d * d, 20, -0.5, 0.5).reshape(d, d), k=unit_rows(hvec(d, 21).reshape(1, d))[0],
                v=hvec(d, 22), beta=np.float32(0.37), decay=np.float32(0.81))


def conv1d_case():
    C = 96
    return dict(C=C, T=5, x=hvec(5 * C, 30).reshape(5, C), w=hvec(4 * C, 31, -0.6, 0.6).reshape(4, C),
                hist=hvec(3 * C, 32).reshape(3, C))


def elementwise_case():
    n = 200
    return dict(a=hvec(n, 40, -6, 6), b=hvec(n, 41, -2, 2))


def rope_case():
    return dict(d_head=256, pos=37, q=hvec(256, 50), k=hvec(256, 51))
