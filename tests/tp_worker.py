"""One tensor-parallel rank of the 2-GPU parity check (launched by test_tp_gpu.py through
torch.distributed.run, one process per GPU; the process group is gloo and only swaps IPC
handles). Rank 0 also builds the single-GPU model and compares greedy ids and logits."""
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    import torch.distributed as dist
    import vkllama_b200 as vk
    from vkllama_b200 import tp as vtp
    from oracle import oracle as O

    os.environ["VKLLAMA_PREFILL"] = "sequential"  # the single-GPU twin prefills token by token too
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo")
    cfg = json.loads(sys.argv[1])
    seed, P, n_gen = cfg.pop("seed"), cfg.pop("prompt"), cfg.pop("n_gen")
    dev = vk.Device(int(os.environ.get("LOCAL_RANK", rank)))
    m = vk.Model(dev, cfg["dim"], cfg["heads"], cfg["ffn"], cfg["vocab"], cfg["layers"], cfg["maxlen"], tp_rank=rank, tp_size=world)
    m.synth_weights(seed)
    vtp.connect(m, dist, rank, world)
    prompt = O.synth_tokens(seed, 1000, P, cfg["vocab"])
    ids, _, _ = m.generate(prompt, n_gen)
    ids2, _, dec_ms = m.generate(prompt, n_gen)  # a second job reuses the exchange buffers
    # one more decode step through the per-token call: every rank returns its logits slice
    logits = m(np.array([ids[-1]], np.uint32), P + n_gen - 1)
    gathered = [None] * world
    dist.all_gather_object(gathered, (ids.tolist(), ids2.tolist(), logits))
    ok = True
    if rank == 0:
        one = vk.Model(dev, cfg["dim"], cfg["heads"], cfg["ffn"], cfg["vocab"], cfg["layers"], cfg["maxlen"])
        one.synth_weights(seed)
        want, _, _ = one.generate(prompt, n_gen)
        want_logits = one(np.array([want[-1]], np.uint32), P + n_gen - 1)
        full = np.concatenate([g[2] for g in gathered])
        same_ranks = all(g[0] == gathered[0][0] and g[1] == gathered[0][0] for g in gathered)
        err = float(np.abs(full - want_logits).max())
        match = ids.tolist() == want.tolist()
        om = O.Model(seed=seed, **cfg)
        oids, gap = om.generate(prompt, n_gen)
        print(json.dumps({"ranks_agree": same_ranks, "ids_match_tp1": match, "logits_max_abs": err,
                          "ids_match_oracle_from_2nd": ids.tolist()[1:] == oids.tolist()[1:],
                          "ids": ids.tolist(), "tp1": want.tolist(), "oracle": oids.tolist(), "ms_per_token": dec_ms / max(1, n_gen - 1)}))
        ok = same_ranks and match and err <= 5e-2
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()
