"""Tensor-parallel decode on 2, 4 and 8 GPUs against the single-GPU model (the parity oracle of
the sharded path: the reference is single-device) — one process per GPU, started like the
benchmark is. Each rank count is skipped when the box has fewer GPUs."""
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


NGPU = _gpus()

# toy models, and the Llama-2-13B geometry cut to two blocks: at 8 ranks 5 heads, 20-block
# column shards of o_proj and 54-block column shards of down per rank
TOY_4 = dict(dim=256, heads=4, ffn=512, vocab=1000, layers=3, maxlen=128, seed=8, prompt=9, n_gen=24)
TOY_8 = dict(dim=512, heads=8, ffn=1024, vocab=2000, layers=2, maxlen=64, seed=9, prompt=1, n_gen=16)
GEOM_13B = dict(dim=5120, heads=40, ffn=13824, vocab=4000, layers=2, maxlen=128, seed=10, prompt=12, n_gen=24)


# the same geometry with a 97-token prompt: 96 tokens in one sharded many-token pass, the last through the decode kernel
MANY_13B = dict(GEOM_13B, maxlen=256, seed=11, prompt=97, n_gen=16, many_token_prefill=True)
MANY_TOY = dict(dim=512, heads=8, ffn=1024, vocab=2000, layers=3, maxlen=256, seed=12, prompt=150, n_gen=12, many_token_prefill=True)


# the all-reduce as an op of its own (the switch VKLLAMA_TP_ALLREDUCE=separate) must keep giving the same ids
TOY_4_SEPARATE = dict(TOY_4, seed=14, allreduce="separate")
# a prompt longer than one many-token pass takes (1024 rows): two passes at different offsets, then the decode kernel
MANY_LONG = dict(dim=512, heads=8, ffn=1024, vocab=2000, layers=2, maxlen=2048, seed=13, prompt=1100, n_gen=8, many_token_prefill=True)


@pytest.mark.parametrize("world", [2, 4, 8])
def test_tp_matches_single_gpu(world):
    if NGPU < world:
        pytest.skip("needs %d GPUs" % world)
    cases = [c for c in (TOY_4, TOY_4_SEPARATE, TOY_8, GEOM_13B, MANY_13B, MANY_TOY, MANY_LONG) if c["heads"] % world == 0]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=%d" % world, "--master-addr", "127.0.0.1",
           "--master-port", str(29610 + world), os.path.join(ROOT, "tests", "tp_worker.py"), json.dumps(cases)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=560, env=env)
    line = [l for l in r.stdout.splitlines() if l.startswith("{")]
    assert line, r.stdout[-2000:] + r.stderr[-2000:]
    res = json.loads(line[-1])
    for c in res["cases"]:
        assert c["ok"], c
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
