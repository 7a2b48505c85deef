"""CPU, 2 gloo ranks: the tensor-parallel sharding rules of the host layer (lb_model_shard_host,
the same code lb_model_load_layer runs) reproduce the unsharded layer: column-parallel shards
concatenate to the full projection, row-parallel partial sums all-reduce to it."""
import os
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent


def _worker(rank, world, port, q):
    sys.path.insert(0, str(ROOT))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    import torch
    import torch.distributed as dist
    import lithos_b200 as lb
    from lithos_b200 import model as M, tp
    from oracle import oracle as orc
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        cfg = M.tiny()
        H = cfg.hidden
        x = lb.fill_normal(H, 3, 1).astype(np.float16)
        for layer in (0, 3):                      # a DeltaNet layer and an attention layer
            slots = M.synthetic_layer_slots(cfg, 11, layer)
            fa = cfg.is_fa(layer)
            # ---- column-parallel: fused input projection
            qw, sc, qz, K, N = tp.shard_host(cfg, rank, world, layer, 0, slots)
            y_shard, _ = orc.gptq_gemv(qw, sc, qz, x, K, N)
            fq, fs, fz, fK, fN = tp.shard_host(cfg, 0, 1, layer, 0, slots)
            y_full, _ = orc.gptq_gemv(fq, fs, fz, x, fK, fN)
            if not fa:
                QK, V = cfg.dn_k_heads * 128, cfg.dn_v_heads * 128
                qk, v = QK // world, V // world
                want = np.concatenate([y_full[rank * qk:(rank + 1) * qk], y_full[QK + rank * qk:QK + (rank + 1) * qk],
                                       y_full[2 * QK + rank * v:2 * QK + (rank + 1) * v],
                                       y_full[2 * QK + V + rank * v:2 * QK + V + (rank + 1) * v]])
            else:
                NQ, NKV = 2 * cfg.fa_q_heads * 256, cfg.fa_kv_heads * 256
                nq = NQ // world
                kv0 = (rank * cfg.fa_kv_heads) // world      # tiny(): 1 KV head shared by both ranks
                want = np.concatenate([y_full[rank * nq:(rank + 1) * nq], y_full[NQ + kv0 * 256:NQ + (kv0 + 1) * 256],
                                       y_full[NQ + NKV + kv0 * 256:NQ + NKV + (kv0 + 1) * 256]])
            assert np.array_equal(y_shard, want), f"layer {layer}: column-parallel shard differs"
            # ---- row-parallel: out / o projection and down projection, partial sums all-reduced
            for which, Kfull in ((1, (cfg.fa_q_heads * 256) if fa else (cfg.dn_v_heads * 128)), (3, cfg.inter)):
                xin = lb.fill_normal(Kfull, 3, 2 + which).astype(np.float16)
                qw, sc, qz, K, N = tp.shard_host(cfg, rank, world, layer, which, slots)
                assert K == Kfull // world and N == H
                part, _ = orc.gptq_gemv(qw, sc, qz, xin[rank * K:(rank + 1) * K], K, N)
                t = torch.from_numpy(part.astype(np.float64))
                dist.all_reduce(t)
                fq, fs, fz, fK, fN = tp.shard_host(cfg, 0, 1, layer, which, slots)
                full, _ = orc.gptq_gemv(fq, fs, fz, xin, fK, fN)
                err = np.max(np.abs(t.numpy() - full)) / np.max(np.abs(full))
                assert err < 1e-5, f"layer {layer} matrix {which}: all-reduced partials differ ({err})"
            # ---- gate|up: interleaved 64-column blocks of this shard's intermediate slice
            qw, sc, qz, K, N = tp.shard_host(cfg, rank, world, layer, 2, slots)
            y, _ = orc.gptq_gemv(qw, sc, qz, x, K, N)
            g_full, _ = orc.gptq_gemv(slots[M.WS["GATE"]], slots[M.WS["GATE"] + 1], slots[M.WS["GATE"] + 2], x, H, cfg.inter)
            u_full, _ = orc.gptq_gemv(slots[M.WS["UP"]], slots[M.WS["UP"] + 1], slots[M.WS["UP"] + 2], x, H, cfg.inter)
            Is = cfg.inter // world
            blocks = y.reshape(-1, 2, 64)
            assert np.array_equal(blocks[:, 0, :].ravel(), g_full[rank * Is:(rank + 1) * Is])
            assert np.array_equal(blocks[:, 1, :].ravel(), u_full[rank * Is:(rank + 1) * Is])
        q.put((rank, "ok"))
    except Exception as e:  # noqa: BLE001
        import traceback
        q.put((rank, traceback.format_exc()))
    finally:
        dist.destroy_process_group()


def test_two_rank_sharding_matches_unsharded(lb, oracle):
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + os.getpid() % 2000
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=240) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    for rank, msg in results:
        assert msg == "ok", f"rank {rank}: {msg}"
