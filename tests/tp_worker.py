"""Run under torchrun (one process per GPU): tensor-parallel decode of the small test model against
the single-GPU result.  Prints 'TP_OK' on rank 0 when tokens and logits agree."""
import os
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))


def main():
    import torch.distributed as dist
    import lithos_b200 as lb
    from lithos_b200 import model as M, tp
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    dist.init_process_group("gloo")
    steps, seed, P0 = 24, 1234, 20
    cfg = M.tiny(max_ctx=64)
    if world == 4:      # the tiny model has 2 key heads: use a 4-way splittable variant
        cfg.dn_k_heads, cfg.dn_v_heads, cfg.fa_q_heads, cfg.fa_kv_heads = 4, 12, 12, 2
    if world == 8:      # 8-way splittable, and like the benchmark's model fewer KV heads (4) than GPUs: each is held by two ranks
        cfg.dn_k_heads, cfg.dn_v_heads, cfg.fa_q_heads, cfg.fa_kv_heads = 8, 24, 24, 4

    def all_gather(b):
        out = [None] * world
        dist.all_gather_object(out, b)
        return out

    ctx = lb.Context(local)
    comm = tp.make_comm(ctx, rank, world, cfg.hidden, all_gather)
    m = M.Model(ctx, cfg, rank, world)
    tp.attach(m, comm)
    m.fill_synthetic(seed)
    m.seed_state(P0, seed)          # every rank takes its heads of ONE seeded state (as bench.py does)
    m.capture()
    dist.barrier()
    m.set_input(5, P0)
    toks = []
    for _ in range(steps):
        m.replay(1)
        toks.append(m.read_next())
    logits = m.logits()
    assert ctx.device_status() == 0
    all_toks = all_gather(toks)
    all_logits = all_gather(logits)
    ok = all(t == all_toks[0] for t in all_toks)
    if rank == 0:
        ref = M.Model(ctx, cfg)
        ref.fill_synthetic(seed)
        ref.seed_state(P0, seed)
        tok, want = 5, []
        for pos in range(P0, P0 + steps):
            tok = ref.decode(tok, pos)
            want.append(tok)
        full = ref.logits()
        got = np.concatenate(all_logits)
        err = float(np.max(np.abs(got - full)) / np.max(np.abs(full)))
        print(f"tp={world} tokens equal across ranks: {ok}; vs single GPU: {toks == want}; logits rel err {err:.2e}", flush=True)
        if ok and toks == want and err < 2e-3:
            print("TP_OK", flush=True)
        ref.close()
    dist.barrier()
    m.close()
    comm.close()
    ctx.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
