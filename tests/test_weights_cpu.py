"""CPU: weight_index.bin, the reference launcher's weight-table file (src/launcher.s:3267-3282): a tiny synthetic model
written by lb_save_weights comes back byte for byte through lb_weight_index_*, and every malformed file is refused with
LB_ERR_IO / LB_ERR_INVALID and a reason (the launcher itself prints a message and carries on with NULL pointers).
Nothing here touches a GPU."""
import struct

import numpy as np
import pytest


def tiny_model(lb):
    from lithos_b200 import model as M
    cfg = M.tiny()
    slots = [M.synthetic_layer_slots(cfg, 3, l) for l in range(cfg.n_layers)]
    return cfg, slots, M.synthetic_globals(cfg, 3)


def write(tmp_path, lb):
    from lithos_b200 import weights as W
    cfg, slots, glob = tiny_model(lb)
    W.save_weights(tmp_path, cfg, slots, glob)
    return cfg, slots, glob


def test_round_trip(tmp_path, lb):
    from lithos_b200 import weights as W
    cfg, slots, glob = write(tmp_path, lb)
    raw = (tmp_path / "weight_index.bin").read_bytes()
    magic, version, n_shards, n_layers, n_slots, n_globals = struct.unpack_from("<6I", raw)
    assert (magic, version, n_shards, n_layers, n_slots, n_globals) == (0x4C575449, 1, 1, cfg.n_layers, 26, 3)
    assert len(raw) == 32 + 264 + (3 + cfg.n_layers * 26) * 24
    w = W.WeightIndex(tmp_path)
    assert w.dims() == (cfg.n_layers, 26, 3, 1)
    w.check(cfg)
    for i, g in enumerate(glob):
        assert np.array_equal(w.entry(-1, i), g.view(np.uint8).ravel())
    for l in range(cfg.n_layers):
        for s in range(26):
            got, want = w.entry(l, s), slots[l][s]
            assert (got is None) == (want is None), (l, s)
            if want is not None:
                assert np.array_equal(got, want.view(np.uint8).ravel()), (l, s)
                assert got.ctypes.data % 64 == 0
    w.close()


def patched(tmp_path, offset, fmt, value):
    p = tmp_path / "weight_index.bin"
    b = bytearray(p.read_bytes())
    struct.pack_into(fmt, b, offset, value)
    p.write_bytes(bytes(b))


def expect(lb, tmp_path, status, word, cfg=None):
    from lithos_b200 import weights as W
    with pytest.raises(lb.LithosError) as e:
        w = W.WeightIndex(tmp_path)
        try:
            w.check(cfg)
        finally:
            w.close()
    assert e.value.status == status and word in str(e.value), str(e.value)


def test_missing_index(tmp_path, lb):
    expect(lb, tmp_path, lb.LB_ERR_IO, "cannot open")


def test_bad_magic(tmp_path, lb):
    write(tmp_path, lb)
    patched(tmp_path, 0, "<I", 0x12345678)
    expect(lb, tmp_path, lb.LB_ERR_IO, "magic")


def test_wrong_version(tmp_path, lb):
    write(tmp_path, lb)
    patched(tmp_path, 4, "<I", 2)
    expect(lb, tmp_path, lb.LB_ERR_IO, "version")


def test_truncated_index(tmp_path, lb):
    write(tmp_path, lb)
    p = tmp_path / "weight_index.bin"
    p.write_bytes(p.read_bytes()[:-40])
    expect(lb, tmp_path, lb.LB_ERR_IO, "truncated")
    p.write_bytes(p.read_bytes()[:20])
    expect(lb, tmp_path, lb.LB_ERR_IO, "header")


def test_shard_index_out_of_range(tmp_path, lb):
    write(tmp_path, lb)
    first_layer_entry = 32 + 264 + 3 * 24
    patched(tmp_path, first_layer_entry, "<I", 7)
    expect(lb, tmp_path, lb.LB_ERR_IO, "names shard 7")


def test_entry_past_shard_and_short_shard(tmp_path, lb):
    write(tmp_path, lb)
    first_layer_entry = 32 + 264 + 3 * 24
    patched(tmp_path, first_layer_entry + 8, "<Q", 1 << 40)
    expect(lb, tmp_path, lb.LB_ERR_IO, "runs past shard")
    write(tmp_path, lb)
    shard = next(p for p in tmp_path.iterdir() if p.name != "weight_index.bin")
    shard.write_bytes(shard.read_bytes()[:-4096])
    expect(lb, tmp_path, lb.LB_ERR_IO, "the index says")


def test_null_required_slot_and_wrong_size(tmp_path, lb):
    cfg, _, _ = write(tmp_path, lb)
    entry = 32 + 264 + 3 * 24 + 24 * 24          # layer 0, slot 24 (input norm): offset and size to zero = NULL
    patched(tmp_path, entry + 8, "<Q", 0)
    patched(tmp_path, entry + 16, "<Q", 0)
    expect(lb, tmp_path, lb.LB_ERR_INVALID, "layer 0 slot 24 is NULL", cfg)
    write(tmp_path, lb)
    patched(tmp_path, entry + 16, "<Q", 100)
    expect(lb, tmp_path, lb.LB_ERR_IO, "layer 0 slot 24 holds 100 bytes", cfg)


def test_index_of_another_model_shape(tmp_path, lb):
    from lithos_b200 import model as M
    write(tmp_path, lb)
    other = M.tiny(n_layers=8)
    expect(lb, tmp_path, lb.LB_ERR_IO, "the model wants 8", other)
