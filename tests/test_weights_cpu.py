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


# ---- safetensors checkpoint -> weight_index.bin (lb_weight_index_from_safetensors) ----
# tensor-name suffixes of the reference's slot table (src/launcher.s:92-141), restated here so that the test does not
# share the library's table
DN = ["linear_attn.in_proj_qkv", "linear_attn.in_proj_z", "linear_attn.out_proj"]
FA = ["self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj", "self_attn.o_proj"]
MLP = ["mlp.gate_proj", "mlp.up_proj", "mlp.down_proj"]
Q4 = ["qweight", "scales", "qzeros"]


def slot_names(cfg, l):
    fa = l % cfg.fa_period == cfg.fa_period - 1
    names = [None] * 26
    if fa:
        for i, p in enumerate(FA):
            for j, q in enumerate(Q4):
                names[3 * i + j] = f"{p}.{q}"
        names[12], names[13] = "self_attn.q_norm.weight", "self_attn.k_norm.weight"
    else:
        for i, p in enumerate(DN):
            for j, q in enumerate(Q4):
                names[3 * i + j] = f"{p}.{q}"
        names[9:15] = ["linear_attn.in_proj_a.weight", "linear_attn.in_proj_b.weight", "linear_attn.A_log", "linear_attn.dt_bias",
                       "linear_attn.conv1d.weight", "linear_attn.norm.weight"]
    for i, p in enumerate(MLP):
        for j, q in enumerate(Q4):
            names[15 + 3 * i + j] = f"{p}.{q}"
    names[24], names[25] = "input_layernorm.weight", "post_attention_layernorm.weight"
    return [n and f"model.layers.{l}.{n}" for n in names]


def write_safetensors(path, tensors, metadata=True):
    """tensors: [(name, uint8 array)] in file order; the dtype/shape fields are what a reader of the index ignores"""
    import json
    head, off = {}, 0
    if metadata:
        head["__metadata__"] = {"format": "pt", "note": 'a "quoted" {brace} ] , in a string'}
    for name, a in tensors:
        head[name] = {"dtype": "U8", "shape": [int(a.size)], "data_offsets": [off, off + int(a.size)]}
        off += int(a.size)
    js = json.dumps(head).encode()
    js += b" " * ((8 - len(js) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(js)))
        f.write(js)
        for _, a in tensors:
            f.write(a.tobytes())


def checkpoint(tmp_path, lb, n_files=2, drop=None):
    cfg, slots, glob = tiny_model(lb)
    tensors = [("model.embed_tokens.weight", glob[0]), ("lm_head.weight", glob[1]), ("model.norm.weight", glob[2])]
    for l in range(cfg.n_layers):
        for name, a in zip(slot_names(cfg, l), slots[l]):
            assert (name is None) == (a is None), (l, name)
            if a is not None:
                tensors.append((name, a))
    tensors = [(n, a.view(np.uint8).ravel()) for n, a in tensors if n != drop]
    rng = np.random.default_rng(5)
    rng.shuffle(tensors)                      # a checkpoint's order is not the slot order
    tensors.append(("model.visual.something.else", np.arange(37, dtype=np.uint8)))  # tensors no slot names are ignored
    per = (len(tensors) + n_files - 1) // n_files
    for i in range(n_files):
        write_safetensors(tmp_path / f"model-{i + 1:05d}-of-{n_files:05d}.safetensors", tensors[i * per:(i + 1) * per], metadata=i == 0)
    return cfg, slots, glob


def test_index_from_safetensors(tmp_path, lb):
    from lithos_b200 import weights as W
    cfg, slots, glob = checkpoint(tmp_path, lb)
    W.index_from_safetensors(tmp_path, cfg)
    w = W.WeightIndex(tmp_path)
    assert w.dims() == (cfg.n_layers, 26, 3, 2)
    w.check(cfg)
    for i, g in enumerate(glob):
        assert np.array_equal(w.entry(-1, i), g.view(np.uint8).ravel())
    for l in range(cfg.n_layers):
        for s in range(26):
            got, want = w.entry(l, s), slots[l][s]
            assert (got is None) == (want is None), (l, s)
            if want is not None:
                assert np.array_equal(got, want.view(np.uint8).ravel()), (l, s)
    w.close()


def test_index_from_safetensors_refusals(tmp_path, lb):
    from lithos_b200 import weights as W
    with pytest.raises(lb.LithosError) as e:      # no checkpoint there
        W.index_from_safetensors(tmp_path, tiny_model(lb)[0])
    assert e.value.status == lb.LB_ERR_IO and "safetensors" in str(e.value)
    cfg, _, _ = checkpoint(tmp_path, lb, n_files=1, drop="model.layers.1.mlp.up_proj.scales")
    with pytest.raises(lb.LithosError) as e:      # a tensor of the slot table is missing
        W.index_from_safetensors(tmp_path, cfg)
    assert e.value.status == lb.LB_ERR_INVALID and "model.layers.1.mlp.up_proj.scales" in str(e.value)
    assert not (tmp_path / "weight_index.bin").exists()
    cfg, _, _ = checkpoint(tmp_path, lb, n_files=1)
    from lithos_b200 import model as M
    other = M.tiny()
    other.inter *= 2                              # the checkpoint is not of this shape
    with pytest.raises(lb.LithosError) as e:
        W.index_from_safetensors(tmp_path, other)
    assert e.value.status == lb.LB_ERR_IO and "bytes" in str(e.value)
    p = tmp_path / "model-00001-of-00001.safetensors"
    raw = p.read_bytes()
    p.write_bytes(struct.pack("<Q", len(raw)) + raw[8:])   # header length past the end of the file
    with pytest.raises(lb.LithosError) as e:
        W.index_from_safetensors(tmp_path, cfg)
    assert e.value.status == lb.LB_ERR_IO and "header length" in str(e.value)
    p.write_bytes(raw[:8] + b"[" + raw[9:])                  # not an object
    with pytest.raises(lb.LithosError) as e:
        W.index_from_safetensors(tmp_path, cfg)
    assert e.value.status == lb.LB_ERR_IO
