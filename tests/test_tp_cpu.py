"""Host logic of the tensor-parallel path on CPU: shard geometry, slicing of 34-byte
block matrices, and the handle exchange over world_size-2 and -4 gloo groups. The exchange step
itself (peer stores inside the decode kernel) needs GPUs: tests/test_tp_gpu.py."""
import os
import subprocess
import sys

import numpy as np

from oracle import oracle as O
import vkllama_b200 as vk
from vkllama_b200 import tp as vtp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = r'''
import os, sys, numpy as np
sys.path.insert(0, sys.argv[1])
import torch, torch.distributed as dist
from oracle import oracle as O
import vkllama_b200 as vk
from vkllama_b200 import tp as vtp
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
dist.init_process_group("gloo")
class Fake:  # stands in for a device model: records what connect() hands it
    def tp_export(self): return bytes([rank]) * 64
    def tp_connect(self, handles): self.handles = handles
f = Fake()
vtp.connect(f, dist, rank, world)
assert [h[0] for h in f.handles] == list(range(world))
# row-split then column-split mat-vec, reduced over the group, equals the full product
N, K = 64, 256
w = O.synth_q8_0(3, 1, N, K); x = O.f16(O.synth_f16(3, 2, K))
full = vk.q8_0_dequantize(w, N, K) @ x
c0, nc = vtp.shard_cols(K, rank, world)
ws = vtp.slice_q8_0(w, N, K, 0, N, c0, nc)
part = torch.from_numpy(vk.q8_0_dequantize(ws, N, nc) @ x[c0:c0 + nc])
dist.all_reduce(part)
assert np.allclose(part.numpy(), full, atol=1e-4), np.abs(part.numpy() - full).max()
r0, nr = vtp.shard_rows(N, rank, world)
rows = vk.q8_0_dequantize(vtp.slice_q8_0(w, N, K, r0, nr, 0, K), nr, K) @ x
out = [torch.zeros(nr, dtype=torch.float32) for _ in range(world)]
dist.all_gather(out, torch.from_numpy(rows.astype(np.float32)))
assert np.allclose(torch.cat(out).numpy(), full, atol=1e-4)
dist.barrier(); dist.destroy_process_group()
print("rank", rank, "ok")
'''


def test_shard_geometry():
    assert vtp.shard_rows(5120, 3, 8) == (1920, 640)
    assert vtp.shard_cols(13824, 7, 8) == (12096, 1728)  # 54 whole blocks per rank
    w = O.synth_q8_0(1, 1, 8, 128)
    s = vtp.slice_q8_0(w, 8, 128, 2, 4, 32, 64)
    full = vk.q8_0_dequantize(w, 8, 128)
    assert np.array_equal(vk.q8_0_dequantize(s, 4, 64), full[2:6, 32:96])


import pytest


@pytest.mark.parametrize("world", [2, 4])
def test_gloo_exchange_and_sharded_matvec(tmp_path, world):
    script = tmp_path / "w.py"
    script.write_text(WORKER)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=%d" % world, "--master-addr", "127.0.0.1",
           "--master-port", str(29613 + world), str(script), ROOT]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-1500:] + r.stderr[-1500:]
    assert r.stdout.count("ok") == world
