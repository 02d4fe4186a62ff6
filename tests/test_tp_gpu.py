"""Tensor-parallel decode on 2 GPUs against the single-GPU model (the parity oracle of the
sharded path: the reference is single-device) — one process per GPU, started like the
benchmark is. Skipped when the box has fewer than 2 GPUs."""
import json
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _gpus():
    try:
        out = subprocess.run(["nvidia-smi", "-L"], capture_output=True, text=True, timeout=30).stdout
        return sum(1 for l in out.splitlines() if l.startswith("GPU "))
    except Exception:
        return 0


@pytest.mark.skipif(_gpus() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("cfg", [
    dict(dim=256, heads=4, ffn=512, vocab=1000, layers=3, maxlen=128, seed=8, prompt=9, n_gen=24),
    dict(dim=512, heads=8, ffn=1024, vocab=2000, layers=2, maxlen=64, seed=9, prompt=1, n_gen=16),
])
def test_tp2_matches_single_gpu(cfg):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29611", os.path.join(ROOT, "tests", "tp_worker.py"), json.dumps(cfg)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=280, env=env)
    line = [l for l in r.stdout.splitlines() if l.startswith("{")]
    assert r.returncode == 0 and line, r.stdout[-2000:] + r.stderr[-2000:]
    res = json.loads(line[-1])
    assert res["ranks_agree"] and res["ids_match_tp1"] and res["logits_max_abs"] <= 5e-2, res
