"""weight_index.bin (the reference launcher's weight-table file, src/launcher.s:3267-3282): host-side mirror of
lb_weight_index_* / lb_save_weights / lb_load_weights.  The index calls need no GPU."""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import LB_OK, LithosError, lib
from .model import ModelCfg, WG_SLOTS, WS_SLOTS

_done = False


def _sigs():
    global _done
    if _done:
        return
    L = lib()
    vp, i32, sz = C.c_void_p, C.c_int, C.c_size_t
    P = C.POINTER
    L.lb_weight_index_open.argtypes = [C.c_char_p, P(vp), C.c_char_p, sz]
    L.lb_weight_index_dims.argtypes = [vp, P(i32), P(i32), P(i32), P(i32)]
    L.lb_weight_index_entry.argtypes = [vp, i32, i32, P(vp), P(sz)]
    L.lb_weight_index_check.argtypes = [vp, P(ModelCfg), C.c_char_p, sz]
    L.lb_weight_index_close.argtypes = [vp]
    L.lb_weight_index_close.restype = None
    L.lb_model_slot_bytes.argtypes = [P(ModelCfg), i32, i32]
    L.lb_model_slot_bytes.restype = sz
    L.lb_model_global_bytes.argtypes = [P(ModelCfg), i32]
    L.lb_model_global_bytes.restype = sz
    L.lb_save_weights.argtypes = [C.c_char_p, P(ModelCfg), P(vp), P(vp), C.c_char_p, sz]
    L.lb_load_weights.argtypes = [vp, C.c_char_p, vp]
    L.lb_weight_index_from_safetensors.argtypes = [C.c_char_p, P(ModelCfg), C.c_char_p, sz]
    _done = True


def slot_bytes(cfg: ModelCfg, layer: int, slot: int) -> int:
    _sigs()
    return lib().lb_model_slot_bytes(C.byref(cfg), layer, slot)


def global_bytes(cfg: ModelCfg, which: int) -> int:
    _sigs()
    return lib().lb_model_global_bytes(C.byref(cfg), which)


def save_weights(model_dir: str, cfg: ModelCfg, layer_slots, globals_) -> None:
    """layer_slots[l][slot] / globals_[i]: numpy arrays (None = unused slot) in the reference's packed formats"""
    _sigs()
    flat = []
    for l in range(cfg.n_layers):
        for s in range(WS_SLOTS):
            a = layer_slots[l][s]
            if a is not None:
                assert a.flags["C_CONTIGUOUS"] and a.nbytes == slot_bytes(cfg, l, s), (l, s, a.nbytes, slot_bytes(cfg, l, s))
            flat.append(a.ctypes.data if a is not None else None)
    arr = (C.c_void_p * len(flat))(*flat)
    g = (C.c_void_p * WG_SLOTS)(*[a.ctypes.data for a in globals_])
    err = C.create_string_buffer(512)
    st = lib().lb_save_weights(str(model_dir).encode(), C.byref(cfg), arr, g, err, 512)
    if st != LB_OK:
        raise LithosError(st, err.value.decode())


def index_from_safetensors(model_dir: str, cfg: ModelCfg) -> None:
    """lb_weight_index_from_safetensors: writes model_dir/weight_index.bin over the *.safetensors files lying there, every
    slot found by the tensor name the reference resolves it from (src/launcher.s:92-141)"""
    _sigs()
    err = C.create_string_buffer(512)
    st = lib().lb_weight_index_from_safetensors(str(model_dir).encode(), C.byref(cfg), err, 512)
    if st != LB_OK:
        raise LithosError(st, err.value.decode())


class WeightIndex:
    """An opened weight_index.bin with its shard files mapped (host only)."""

    def __init__(self, model_dir: str):
        _sigs()
        self.h = C.c_void_p(None)
        err = C.create_string_buffer(512)
        st = lib().lb_weight_index_open(str(model_dir).encode(), C.byref(self.h), err, 512)
        if st != LB_OK:
            raise LithosError(st, err.value.decode())

    def dims(self):
        v = [C.c_int(0) for _ in range(4)]
        lib().lb_weight_index_dims(self.h, *[C.byref(x) for x in v])
        return tuple(x.value for x in v)   # layers, slots per layer, globals, shards

    def entry(self, layer: int, slot: int):
        """bytes of (layer, slot) as a uint8 view of the mapping (None when unused); layer < 0: global `slot`"""
        p, n = C.c_void_p(None), C.c_size_t(0)
        st = lib().lb_weight_index_entry(self.h, layer, slot, C.byref(p), C.byref(n))
        if st != LB_OK:
            raise LithosError(st, "weight index: no such entry")
        if not p.value:
            return None
        return np.ctypeslib.as_array(C.cast(p, C.POINTER(C.c_uint8)), shape=(n.value,))

    def check(self, cfg: ModelCfg) -> None:
        err = C.create_string_buffer(512)
        st = lib().lb_weight_index_check(self.h, C.byref(cfg), err, 512)
        if st != LB_OK:
            raise LithosError(st, err.value.decode())

    def close(self):
        if self.h:
            lib().lb_weight_index_close(self.h)
            self.h = None


def load_weights(model, model_dir: str) -> None:
    """lb_load_weights: index -> shards -> every layer and the globals of `model` (a lithos_b200.model.Model)"""
    _sigs()
    model.ctx._check(lib().lb_load_weights(model.ctx.h, str(model_dir).encode(), model.h))
