"""One tensor-parallel rank of the multi-GPU parity check (launched by test_tp_gpu.py through
torch.distributed.run, one process per GPU; the process group is gloo and only swaps IPC
handles). Every case in the JSON list of argv[1] is run in turn. Rank 0 also builds the
single-GPU model, which is the parity oracle of the sharded path (the reference is
single-device), walks it token by token to get its ids and top-2 logit gaps, and compares."""
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

UNDECIDED_ULPS = 4.0  # a step the single-GPU model decides by less than this may legitimately differ


def gap_ulps(logits):
    top = int(np.argmax(logits))
    v = float(logits[top])
    second = float(np.max(np.delete(logits, top)))
    ulp = 2.0 ** (np.floor(np.log2(max(abs(v), 2.0 ** -14))) - 10)
    return top, (v - second) / ulp


def run_case(cfg, dist, rank, world, vk, vtp, synth_tokens):
    cfg = dict(cfg)
    seed, P, n_gen = cfg.pop("seed"), cfg.pop("prompt"), cfg.pop("n_gen")
    dev = vk.Device(int(os.environ.get("LOCAL_RANK", rank)))
    m = vk.Model(dev, cfg["dim"], cfg["heads"], cfg["ffn"], cfg["vocab"], cfg["layers"], cfg["maxlen"], tp_rank=rank, tp_size=world)
    m.synth_weights(seed)
    vtp.connect(m, dist, rank, world)
    prompt = synth_tokens(seed, 1000, P, cfg["vocab"])
    # "many_token_prefill": all but the last prompt token go through the sharded many-token pass (tensor-core
    # GEMMs, partial sums of the K-split projections summed over the ranks); the twin then prefills the same way
    many = cfg.pop("many_token_prefill", False)
    # "allreduce": "separate" keeps the all-reduce as an op of its own behind the K-split projections (the decode
    # plan reads the switch when it is built, at the first one-token step)
    if cfg.pop("allreduce", "in place") == "separate":
        os.environ["VKLLAMA_TP_ALLREDUCE"] = "separate"
    else:
        os.environ.pop("VKLLAMA_TP_ALLREDUCE", None)
    if many:
        os.environ.pop("VKLLAMA_PREFILL", None)
    else:
        os.environ["VKLLAMA_PREFILL"] = "sequential"
    n0 = vk.kernel_launches()
    ids, _, _ = m.generate(prompt, n_gen)
    launches = vk.kernel_launches() - n0
    ids2, _, dec_ms = m.generate(prompt, n_gen)  # a second job reuses the exchange buffers
    # one more decode step through the per-token call: every rank returns its logits slice
    logits = m(np.array([ids[-1]], np.uint32), P + n_gen - 1)
    # a several-token call on the sharded model (the reference's Model::operator() with a prompt): every rank's
    # slice of the last token's logits, against the twin fed the same tokens with its last one in a call of its own
    multi = None
    if many:
        k = P - 7
        multi = m(prompt[:k], 0)
    gathered = [None] * world
    dist.all_gather_object(gathered, (ids.tolist(), ids2.tolist(), logits, multi))
    res = None
    if rank == 0:
        one = vk.Model(dev, cfg["dim"], cfg["heads"], cfg["ffn"], cfg["vocab"], cfg["layers"], cfg["maxlen"])
        one.synth_weights(seed)
        # the single-GPU twin, token by token like the sharded model prefills
        if many:
            one(prompt[:P - 1], 0)
            lg = one(prompt[P - 1:], P - 1)
        else:
            for i in range(P):
                lg = one(np.array([prompt[i]], np.uint32), i)
        want, gaps = [], []
        for i in range(n_gen):
            if i:
                lg = one(np.array([want[-1]], np.uint32), P + i - 1)
            top, g = gap_ulps(lg)
            want.append(top)
            gaps.append(g)
        # teacher-forced logits at the sharded model's own last position
        one2_logits = None
        if ids.tolist() == want:
            one2_logits = one(np.array([want[-1]], np.uint32), P + n_gen - 1)
        multi_err = None
        if many:
            k = P - 7
            one(prompt[:k - 1], 0)
            want_multi = one(prompt[k - 1:k], k - 1)
            multi_err = float(np.abs(np.concatenate([g[3] for g in gathered]) - want_multi).max())
        full = np.concatenate([g[2] for g in gathered])
        same_ranks = all(g[0] == gathered[0][0] and g[1] == gathered[0][0] for g in gathered)
        bad = [i for i in range(n_gen) if ids[i] != want[i]]
        follows = (not bad) or gaps[bad[0]] < UNDECIDED_ULPS
        err = float(np.abs(full - one2_logits).max()) if one2_logits is not None else None
        res = {"cfg": cfg, "world": world, "ranks_agree": same_ranks, "ids_match_tp1": not bad, "follows_tp1_to_first_undecided_step": follows,
               "first_mismatch": bad[0] if bad else None, "gap_ulps_there": gaps[bad[0]] if bad else None,
               "min_gap_ulps": min(gaps), "logits_max_abs": err, "ms_per_token": dec_ms / max(1, n_gen - 1)}
        res["ok"] = bool(same_ranks and follows and (bad or err <= 5e-2) and (not bad or bad[0] >= 2))
        if many:  # the pass really ran: a few kernels per block instead of one launch per prompt token
            res["launches"] = launches
            res["multi_token_call_logits_max_abs"] = multi_err
            res["ok"] = bool(res["ok"] and launches < P and multi_err <= 5e-2)
        one.close()
    dist.barrier()
    m.close()
    dev.close()
    return res


def main():
    import torch.distributed as dist
    import vkllama_b200 as vk
    from vkllama_b200 import tp as vtp
    from vkllama_b200.synth import synth_tokens

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo")
    cases = json.loads(sys.argv[1])
    out = [run_case(c, dist, rank, world, vk, vtp, synth_tokens) for c in cases]
    ok = True
    if rank == 0:
        print(json.dumps({"world": world, "cases": out}))
        ok = all(r["ok"] for r in out)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()
