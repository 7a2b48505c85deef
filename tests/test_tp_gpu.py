"""GPU (needs >= 2 GPUs on the box; skipped otherwise): tensor-parallel decode through IPC-mapped
exchange buffers gives the same greedy tokens as one GPU, and logits within 2e-3 of max|logit| (the shards quantise their
activation slices separately and add partial sums in a different order).  Worlds 2, 4 and 8; the recurrent state and a KV
prefix are seeded from ONE global state of which every rank takes its heads.  (On a one-GPU box the same parity is
visible in bench.py's `parity.first_tokens`, which must be the same list at every N.)"""
import os
import subprocess
import sys
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def _gpu_count():
    try:
        out = subprocess.run(["nvidia-smi", "-L"], capture_output=True, text=True, timeout=30).stdout
        n = sum(1 for l in out.splitlines() if l.startswith("GPU "))
        vis = os.environ.get("CUDA_VISIBLE_DEVICES")          # a restricted process sees fewer than the box has
        return min(n, len([v for v in vis.split(",") if v.strip()])) if vis is not None else n
    except Exception:  # noqa: BLE001
        return 0


@pytest.mark.parametrize("world", [2, 4, 8])
def test_tp_decode_matches_single_gpu(world):
    if _gpu_count() < world:
        pytest.skip(f"needs {world} GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
                        "--master-addr", "127.0.0.1", "--master-port", str(29600 + world), str(ROOT / "tests" / "tp_worker.py")],
                       capture_output=True, text=True, timeout=600, env=env)
    assert "TP_OK" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]
