#!/usr/bin/env python
"""Headline benchmark: Llama-2-7B Q8_0 batch-1 greedy decode tokens/s on one B200
(and Llama-2-13B Q8_0 tensor-parallel at 2/4/8 GPUs), with the HBM roofline of
the weight-plus-KV stream beside it and the CPU port timed on the host cores.

    python bench.py --gpus 1 --steps K --warmup W            # this library
    python bench.py --impl reference --steps K --warmup W    # CPU port of the reference's op math

One step = one whole job of the workload: prefill of the seeded prompt, then
the greedy decode tokens, each decode token one launch of the persistent decode
kernel. `value` is decoded tokens per second over the decode phases (the
reference's "eval speed", app/llama2_infer.cpp:212-218), timed with CUDA events
on the stream the kernel is launched on. Weights are synthetic (seeded N(0,0.02),
Q8_0-quantised on the device): no checkpoint is read.

Every line carries `parity`: a hash of the first greedy ids of the timed job, whether all
ranks produced the same ids, and (13B) how far the ids follow the single-GPU model's, which
rank 0 runs beside the sharded one. The 1-GPU line also carries `tp_anchor`: the 13B model on
one GPU, the base of the 2/4/8-GPU curve.
"""
import argparse
import hashlib
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# Tensor ids of the seeded prompts. They were picked by tests/golden/screen_prompts_gpu.py so that the
# first PARITY_IDS greedy steps are each decided by several fp16 ulps: implementations that differ
# only in fp32 summation order (decode plans, tensor-parallel degrees) then produce the same ids,
# and `parity.ids_sha` can be compared across lines.
PROMPT_ID_7B = 3144    # smallest top-2 gap over 64 steps: 14 fp16 ulps (32-token prompt, one multi-token call)
PROMPT_ID_13B = 2037   # 7 fp16 ulps over 64 steps (128-token prompt fed token by token)
PARITY_IDS = 64

WORKLOADS = {
    # name: dims, prompt, decode tokens
    "llama2-7b-q8_0": dict(dim=4096, heads=32, ffn=11008, vocab=32000, layers=32, maxlen=4096,
                           prompt=32, decode=256, seed=20240602, prompt_id=PROMPT_ID_7B),
    "llama2-13b-q8_0": dict(dim=5120, heads=40, ffn=13824, vocab=32000, layers=40, maxlen=4096,
                            prompt=128, decode=512, seed=20240604, prompt_id=PROMPT_ID_13B),
    # FP16 weights, 512-token prompt: the prefill runs on the tcgen05 tensor-core GEMMs (a parity/profiling case, not the headline)
    "llama2-7b-f16": dict(dim=4096, heads=32, ffn=11008, vocab=32000, layers=32, maxlen=4096,
                          prompt=512, decode=256, seed=20240603, weights="f16"),
    # 4 of the 32 blocks of the 7B shape: the small case for multi-pass ncu captures (1.2 GB on the device)
    "llama2-7b-q8_0-4blocks": dict(dim=4096, heads=32, ffn=11008, vocab=32000, layers=4, maxlen=4096,
                                   prompt=32, decode=16, seed=20240602),
}


def q8_bytes(rows, cols):
    return rows * (cols // 32) * 34


def bytes_per_token(w, L, tp=1):
    """Algorithmic HBM bytes of one decode token at KV length L (after append), per GPU."""
    d, f, v, nl = w["dim"], w["ffn"], w["vocab"], w["layers"]
    wb = (lambda r, c: r * c * 2) if w.get("weights") == "f16" else q8_bytes
    mats = nl * (4 * wb(d, d) + 3 * wb(f, d)) + wb(v, d)
    norms = (2 * nl + 1) * d * 4
    emb = wb(1, d)
    kv = 2 * d * 2 * nl  # K and V, fp16, all heads, all layers, per cached position
    return mats / tp + norms + emb + kv * (L + 1) / tp


def config_of(name, w, world):
    """The `config` object of a line: the same for both arms, so the lines can be compared."""
    Ls = np.arange(w["prompt"] + 1, w["prompt"] + w["decode"] + 1)
    bytes_tok = float(np.mean([bytes_per_token(w, L, world) for L in Ls]))
    return {"workload": name, "batch": 1, "prompt_tokens": w["prompt"], "decode_tokens": w["decode"],
            "kv_len": "%d..%d" % (w["prompt"] + 1, w["prompt"] + w["decode"]),
            "parallelism": "tp%d" % world, "l2": "inputs (%.1f GB of weights per token) larger than L2" % (bytes_tok / 1e9),
            "step": "one job = prefill + %d decode tokens; value counts decode tokens over decode time" % w["decode"]}


def ids_sha(ids):
    """Short sha256 over the first PARITY_IDS greedy ids (uint32, little endian)."""
    return hashlib.sha256(np.asarray(ids[:PARITY_IDS], "<u4").tobytes()).hexdigest()[:16]


def peak_hbm():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


def peak_tensor():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["bf16_tflops"]), "measured"
        except Exception:
            pass
    return 1590.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index=0):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q, "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm, mx, reasons = [], None, set()
        for r in self.rows:
            try:
                sm.append(float(r[0]))
                mx = float(r[1])
                for name, col in (("hw_slowdown", 4), ("hw_thermal_slowdown", 5), ("sw_thermal_slowdown", 6), ("sw_power_cap", 7)):
                    if r[col].lower().startswith("active"):
                        reasons.add(name)
            except Exception:
                pass
        sm.sort()
        load = sm[len(sm) // 2:] if sm else []  # upper half = samples under load
        return {"sm_mhz": (load[len(load) // 2] if load else None), "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm)}


def cpu_port_sample(w, layers_sample=2, steps=16):
    """One bounded sample of the CPU port (oracle): `steps` decode steps through `layers_sample`
    decoder blocks of the workload's shape at mid-range KV length, plus the output layer. Returns
    a closure that runs the sample once and gives (seconds for the sample, seconds per token
    EXTRAPOLATED to the full model: layers / layers_sample x block time + output-layer time)."""
    from oracle import oracle as O
    O.set_threads(os.cpu_count() or 1)  # a launcher may have pinned OMP_NUM_THREADS to 1
    om = O.Model(dim=w["dim"], heads=w["heads"], ffn=w["ffn"], vocab=w["vocab"], layers=layers_sample,
                 maxlen=512, seed=w["seed"])
    L0 = w["prompt"] + w["decode"] // 2
    x = O.synth_f16(w["seed"], 999, w["dim"]).reshape(1, w["dim"])
    # fill the caches so the attention reads a realistic history length
    for l in range(layers_sample):
        om.kcache(l)[:, :L0] = O.synth_f16(w["seed"], 900 + l, w["heads"] * L0 * (w["dim"] // w["heads"])).reshape(w["heads"], L0, -1)
        om.vcache(l)[:, :L0] = om.kcache(l)[:, :L0]
    tok = np.array([1], np.uint32)

    def run():
        a = time.time()
        for n in range(steps):
            for l in range(layers_sample):
                om.block(l, x, 1, L0 + 1 + (n % 8))
        t_block = (time.time() - a) / (steps * layers_sample)
        b = time.time()
        k = max(2, steps // 4)
        for i in range(k):  # whole small model = layers_sample blocks + output layer; the head is the difference
            om.forward(tok, L0 + 10 + i)
        t_fwd = (time.time() - b) / k
        t_head = max(t_fwd - layers_sample * t_block, 0.0)
        return time.time() - a, w["layers"] * t_block + t_head

    what = ("EXTRAPOLATED from a sample: %d of %d decoder blocks + output layer, %d decode steps at KV length ~%d per step, "
            "block time scaled to %d blocks" % (layers_sample, w["layers"], steps, L0, w["layers"]))
    return run, O.threads(), what


def cpu_port_tokens_per_s(w, reps=2):
    run, threads, what = cpu_port_sample(w)
    run()
    per_tok = min(run()[1] for _ in range(reps))
    return 1.0 / per_tok, threads, what


def run_reference(args, w, name):
    """The reference arm: the CPU port of the reference's op math on all host threads. One step is
    one bounded sample (see cpu_port_sample); `value` is tokens/s extrapolated to the full model,
    `ms_per_step` the measured duration of a sample step."""
    run, threads, what = cpu_port_sample(w)
    for _ in range(max(args.warmup, 1)):
        run()
    t_steps, per_tok = [], []
    for _ in range(max(args.steps, 1)):
        t, pt = run()
        t_steps.append(t)
        per_tok.append(pt)
    v = 1.0 / float(np.mean(per_tok))
    line = {"impl": "reference", "metric": "decode_tokens_per_s", "value": v, "unit": "tokens/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1000.0 * float(np.mean(t_steps)), "higher_is_better": True,
            "scaling": "strong" if args.gpus > 1 else "weak", "vs_baseline": None, "dtype": "q8_0 weights, fp16 activations, fp32 accumulate",
            "data": "synthetic", "config": config_of(name, w, args.gpus),
            "cpu_baseline": {"value": v, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": what},
            "e2e": {"value": v, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "note": "the reference runs only through Vulkan (unavailable on this box) and ships no CPU implementation of its ops; "
                    "this arm times the CPU restatement of its shader math (oracle/) on the host cores; value is extrapolated "
                    "from the sample, ms_per_step is the measured time of one sample step"}
    print(json.dumps(line))


# dram__bytes_read.sum + dram__bytes_write.sum of one decode_mega_kernel launch from ncu (see profiles/), per workload
TRAFFIC_NCU = {"llama2-7b-q8_0": 7.06e9}  # 1.005 x algorithmic, scaled from the 4-block capture (profiles/decode_mega_kernel_7b_shape_4blocks.md)

MICRO_SHAPES = [(4096, 4096), (11008, 4096), (4096, 11008), (32000, 4096)]  # rows x K: qkvo, gate/up, down, lm head


def run_micro(args):
    """Q8_0 mat-vec / skinny mat-mul microbenchmark through the MatMul op: achieved HBM
    GB/s per weight shape and token count. Weight copies are rotated so that every timed
    launch streams a matrix that is not in L2 (copies total >= 3 x 126 MB)."""
    import vkllama_b200 as vk
    peak, peak_kind = peak_hbm()
    dev = vk.Device(0)
    cmd = vk.Command(dev)
    shapes = MICRO_SHAPES if args.micro == "all" else [tuple(int(v) for v in args.micro.split("x"))]
    tokens = [int(v) for v in args.micro_tokens.split(",")]
    rows = []
    launches0 = vk.kernel_launches()
    for (N, K) in shapes:
        wbytes = q8_bytes(N, K)
        copies = max(2, -(-400_000_000 // wbytes))
        cmd.begin()
        ws = []
        for i in range(copies):
            t = vk.Tensor(1, N, K, dev, vk.Q8_0)
            cmd.fill_synthetic(t, 20240605, i, 0.0, 0.02)
            ws.append(t)
        ops = [vk.MatMul(dev, cmd, t, 1.0, 0.0, 0, 0, True, vk.FP16, vk.Q8_0).init() for t in ws]
        cmd.end()
        cmd.submit_and_wait()
        for M in tokens:
            cmd.begin()
            x = vk.Tensor(1, M, K, dev, vk.FP16)
            cmd.fill_synthetic(x, 20240605, 100 + M, 0.0, 1.0)
            vk.matmul_run_many(ops, x, max(args.warmup, 3) * len(ops))
            cmd.end()
            cmd.submit_and_wait()
            cmd.begin()
            n = args.steps * len(ops)
            us = vk.matmul_run_many(ops, x, n, timed=True)  # one CUDA graph of n launches: device time, no host gaps
            cmd.end()
            cmd.submit_and_wait()
            algo = wbytes + M * K * 2 + M * N * 2
            gbs = algo / (us * 1e-6) / 1e9
            rows.append({"rows": N, "K": K, "tokens": M, "us_per_launch": us, "bytes_per_launch": algo, "GBps": gbs,
                         "frac_of_peak": gbs / peak, "tflops": 2.0 * M * N * K / (us * 1e-6) / 1e12})
        del ops, ws
    print(json.dumps({"metric": "q8_0_matvec_GBps", "unit": "GB/s", "peak": peak, "peak_kind": peak_kind, "steps": args.steps,
                      "timing": "CUDA events around one CUDA graph of steps x copies MatMul op calls (each call = event, kernel, event; no host work between them) over rotated weight copies larger than L2",
                      "gpu_launches": int(vk.kernel_launches() - launches0), "results": rows}))


def run_gemm(args):
    """FP16 prefill GEMM microbenchmark through the MatMul op (MxNxK, weights [N,K]): achieved
    TFLOP/s of the tcgen05 kernel against the measured dense-GEMM peak."""
    import vkllama_b200 as vk
    M, N, K = (int(v) for v in args.gemm.split("x"))
    tpeak, tkind = peak_tensor()
    dev = vk.Device(0)
    cmd = vk.Command(dev)
    q8 = args.gemm_weights == "q8_0"
    wdt = vk.Q8_0 if q8 else vk.FP16
    wbytes = q8_bytes(N, K) if q8 else 2 * N * K
    # weight copies are rotated so that every launch streams a matrix that is not in L2
    copies = max(2, -(-400_000_000 // wbytes))
    a = vk.Tensor(1, M, K, dev, vk.FP16)
    cmd.begin()
    cmd.fill_synthetic(a, 20240606, 1, 0.0, 1.0)
    ws = []
    for i in range(copies):
        wt = vk.Tensor(1, N, K, dev, wdt)
        cmd.fill_synthetic(wt, 20240606, 2 + i, 0.0, 0.02)
        ws.append(wt)
    ops = [vk.MatMul(dev, cmd, wt, 1.0, 0.0, 0, 0, True, vk.FP16, wdt).init() for wt in ws]
    cmd.end()
    cmd.submit_and_wait()
    cmd.begin()
    vk.matmul_run_many(ops, a, max(args.warmup, 3) * len(ops))
    cmd.end()
    cmd.submit_and_wait()
    launches0 = vk.kernel_launches()
    cmd.begin()
    us = vk.matmul_run_many(ops, a, args.steps * len(ops), timed=True)
    cmd.end()
    cmd.submit_and_wait()
    tf = 2.0 * M * N * K / (us * 1e-6) / 1e12
    hpeak, hkind = peak_hbm()
    algo = wbytes + 2 * M * K + 2 * M * N
    gbs = algo / (us * 1e-6) / 1e9
    # which roof is lower for this shape: streaming the weights once, or the dense fp16 tensor rate
    t_hbm, t_tensor = algo / (hpeak * 1e9), 2.0 * M * N * K / (tpeak * 1e12)
    roof = ({"bound": "hbm", "achieved": gbs, "peak": hpeak, "unit": "GB/s", "frac": gbs / hpeak, "peak_kind": hkind}
            if t_hbm > t_tensor else
            {"bound": "tensor", "achieved": tf, "peak": tpeak, "unit": "TFLOP/s", "frac": tf / tpeak, "peak_kind": tkind})
    roof["kernel"] = "gemm_tcgen05_kernel"
    print(json.dumps({"metric": "prefill_gemm_tflops", "value": tf, "unit": "TFLOP/s", "n_gpus": 1, "steps": args.steps,
                      "warmup": max(args.warmup, 3), "us_per_launch": us, "GBps": gbs,
                      "dtype": ("q8_0 (dequantised to fp16 in shared memory)" if q8 else "fp16") + " x fp16 -> fp32 accumulate -> fp16",
                      "config": {"workload": "gemm %dx%dx%d (rows x weight rows x K), %s weights, %d rotated copies" % (M, N, K, args.gemm_weights, copies)},
                      "roofline": roof, "gpu_launches": int(vk.kernel_launches() - launches0)}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--micro", default=None, help="'all' or ROWSxK: Q8_0 mat-vec microbenchmark instead of the token loop")
    ap.add_argument("--micro-tokens", default="1,2,4,8,16,64")
    ap.add_argument("--gemm", default=None, help="MxNxK: tensor-core prefill GEMM microbenchmark instead of the token loop")
    ap.add_argument("--gemm-weights", default="f16", choices=["f16", "q8_0"])
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=None, choices=[None] + list(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-anchor", action="store_true", help="skip the single-GPU 13B model run beside the timed workload")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    name = args.workload or ("llama2-7b-q8_0" if args.gpus == 1 else "llama2-13b-q8_0")
    w = WORKLOADS[name]

    if args.impl == "reference":
        if rank == 0:
            run_reference(args, w, name)
        return 0
    if args.micro:
        if rank == 0:
            run_micro(args)
        return 0
    if args.gemm:
        if rank == 0:
            run_gemm(args)
        return 0

    import vkllama_b200 as vk
    from vkllama_b200.synth import synth_tokens

    tp = world
    dist = None
    if tp > 1:
        import torch
        import torch.distributed as dist
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    dev = vk.Device(local_rank)
    f16w = w.get("weights") == "f16"
    model = vk.Model(dev, w["dim"], w["heads"], w["ffn"], w["vocab"], w["layers"], w["maxlen"],
                     weight_dtype=vk.FP16 if f16w else vk.Q8_0, tp_rank=rank, tp_size=tp)
    model.synth_weights(w["seed"])
    if tp > 1:
        from vkllama_b200 import tp as vtp
        vtp.connect(model, dist, rank, world)
    prompt = synth_tokens(w["seed"], w.get("prompt_id", 1000), w["prompt"], w["vocab"])
    n_gen = w["decode"] + 1  # the prefill yields the first id, then `decode` one-token steps

    def barrier():
        if dist is not None:
            import torch
            dist.barrier()
            torch.cuda.synchronize()

    for _ in range(args.warmup):
        model.generate(prompt, n_gen)
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    launches0 = vk.kernel_launches()
    dec_ms, pre_ms = [], []
    t0 = time.time()
    ids = None
    for _ in range(args.steps):
        ids, p_ms, d_ms = model.generate(prompt, n_gen)  # synchronises its stream before returning
        dec_ms.append(d_ms)
        pre_ms.append(p_ms)
    barrier()
    wall = time.time() - t0
    launches = vk.kernel_launches() - launches0
    clocks = sampler.stop() if rank == 0 else None
    dec_total = float(sum(dec_ms))
    job_ms = float(sum(dec_ms) + sum(pre_ms)) / args.steps
    parity = {"n_ids": PARITY_IDS, "ids_sha": ids_sha(ids), "ranks_agree": True,
              "what": "sha256 over the first %d greedy ids of the last timed job" % PARITY_IDS}
    if dist is not None:
        import torch
        t = torch.tensor([dec_total, job_ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dec_total, job_ms = float(t[0]), float(t[1])
        mine = torch.tensor(np.asarray(ids, np.int64), device="cuda")
        every = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(every, mine)
        parity["ranks_agree"] = bool(all(torch.equal(e, mine) for e in every))  # over all generated ids
    tok_s = args.steps * w["decode"] / (dec_total / 1000.0)
    ms_tok = dec_total / (args.steps * w["decode"])

    # ---- end to end through the reference-facing call: host token ids in, fp32 logits out, host arg-max
    e2e_jobs = min(args.steps, 2)
    e2e_t = 0.0
    for _ in range(e2e_jobs):
        if tp == 1:
            logits = model(prompt, 0)
            tok = np.array([int(np.argmax(logits))], np.uint32)
        else:  # sharded models prefill inside generate; every rank gets the same first id
            first, _, _ = model.generate(prompt, 1)
            tok = np.array([int(first[0])], np.uint32)
        barrier()
        buf = np.empty(w["vocab"] // tp, np.float32)  # the loop's logits buffer, reused every token
        a = time.time()
        for i in range(w["decode"]):
            logits = model(tok, w["prompt"] + i, out=buf)  # this rank's slice of the fp32 logits comes back to the host
            tok[0] = int(np.argmax(logits)) if tp == 1 else model.last_token()
        barrier()
        e2e_t += time.time() - a
    e2e = e2e_jobs * w["decode"] / e2e_t
    prof = np.zeros(20)
    reps = 16
    for i in range(reps):  # collective under tensor parallelism: every rank runs it
        prof += np.array(model.decode_profile(int(prompt[i % len(prompt)]), w["prompt"] + 100 + i))
    prof /= reps
    barrier()

    # ---- the single-GPU 13B model beside the sharded one (rank 0): the parity oracle of tensor
    # parallelism (the reference is single-device) and, on the 1-GPU line, the base of the curve
    anchor = None
    want_anchor = (not args.no_anchor) and rank == 0 and (tp > 1 or name == "llama2-7b-q8_0")
    if want_anchor:
        model.close() if tp == 1 else None
        aw = WORKLOADS["llama2-13b-q8_0"]
        one = vk.Model(dev, aw["dim"], aw["heads"], aw["ffn"], aw["vocab"], aw["layers"], aw["maxlen"])
        one.synth_weights(aw["seed"])
        ap = synth_tokens(aw["seed"], aw["prompt_id"], aw["prompt"], aw["vocab"])
        one.generate(ap, aw["decode"] + 1)
        a_ids, a_pre, a_dec = one.generate(ap, aw["decode"] + 1)
        # the ids the sharded runs are compared with: prompt fed token by token. Sharded models take the last
        # prompt token through the decode kernel; a single-GPU multi-token call instead rotates the last block's
        # clipped query at the call's first position, as the reference does, and its first ids differ for that
        os.environ["VKLLAMA_PREFILL"] = "sequential"
        s_ids, _, _ = one.generate(ap, aw["decode"] + 1)
        os.environ.pop("VKLLAMA_PREFILL", None)
        one.close()
        anchor = {"workload": "llama2-13b-q8_0", "tp": 1, "value": aw["decode"] / (a_dec / 1000.0), "unit": "tokens/s",
                  "ms_per_token": a_dec / aw["decode"], "prefill_ms": a_pre, "ids_sha": ids_sha(s_ids), "n_ids": PARITY_IDS,
                  "ids_sha_what": "token-by-token prefill, comparable with the ids_sha of the 2/4/8-GPU lines",
                  "ids_sha_batched_prefill": ids_sha(a_ids)}
        if tp > 1:
            same = np.asarray(s_ids) == np.asarray(ids)
            parity["tp1"] = {"ids_sha": anchor["ids_sha"], "matches_tp1": anchor["ids_sha"] == parity["ids_sha"],
                             "ids_equal_until": int(np.argmin(same)) if not same.all() else int(same.size),
                             "of": int(same.size)}
    barrier()

    if rank != 0:
        if dist is not None:
            dist.barrier()
            dist.destroy_process_group()
        return 0
    # ---- roofline: whole decode step and the dominant kernel (gate/up mat-vec), live
    peak, peak_kind = peak_hbm()
    Ls = np.arange(w["prompt"] + 1, w["prompt"] + w["decode"] + 1)
    bytes_tok = float(np.mean([bytes_per_token(w, L, tp) for L in Ls]))
    step_gbs = bytes_tok / (ms_tok * 1e-3) / 1e9
    persistent = os.environ.get("VKLLAMA_DECODE", "") != "graph" and prof[10:].sum() > 0
    if persistent:
        # one kernel launch per token: the dominant kernel is the whole decode step
        kname = "decode_mega_kernel (persistent decode step: TMA weight ring + mma.sync consumers, all ops of a token)"
        k_bytes, k_us = bytes_tok, ms_tok * 1e3
    else:
        kname = "mv_kernel (RMSNorm + gate/up %s mat-vec + SwiGLU)" % ("FP16" if f16w else "Q8_0")
        k_bytes = 2 * (w["ffn"] // tp * w["dim"] * 2 if f16w else q8_bytes(w["ffn"] // tp, w["dim"])) + w["dim"] * 2 + w["dim"] * 4 + (w["ffn"] // tp) * 2
        k_us = prof[4] / w["layers"]
    k_gbs = k_bytes / (k_us * 1e-6) / 1e9
    classes = ["embedding", "norm_qkv", "attention", "o_proj_add", "norm_gateup_swiglu", "down_add", "norm_lm_head", "argmax", "allreduce"]
    line = {
        "metric": "decode_tokens_per_s", "value": tok_s, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": job_ms, "higher_is_better": True,
        "scaling": "strong" if world > 1 else "weak", "vs_baseline": None,
        "dtype": "%s weights, fp16 activations, fp32 accumulate" % ("fp16" if f16w else "q8_0"), "data": "synthetic",
        "config": config_of(name, w, world),
        "ms_per_token": ms_tok, "prefill_ms": float(np.mean(pre_ms)),
        "roofline": {"bound": "hbm", "kernel": kname, "achieved": k_gbs,
                     "peak": peak, "unit": "GB/s", "frac": k_gbs / peak, "traffic": TRAFFIC_NCU.get(name) if persistent else None,
                     "peak_kind": peak_kind, "bytes_per_launch": k_bytes, "us_per_launch": k_us},
        "roofline_step": {"bound": "hbm", "what": "whole decode token: weights + norm weights + embedding row + KV", "achieved": step_gbs,
                          "peak": peak, "unit": "GB/s", "frac": step_gbs / peak, "frac_of_8TBs_nominal": step_gbs / 8000.0,
                          "bytes_per_token": bytes_tok, "peak_kind": peak_kind},
        "op_us_per_token": dict(zip(classes, [float(x) for x in prof[:9]])),
        "op_wait_us_per_token": dict(zip(classes, [float(x) for x in prof[10:19]])),
        "decode_path": "persistent kernel" if persistent else "cuda graph of 5 kernels per layer",
        "e2e": {"value": e2e, "unit": "tokens/s", "h2d_bytes_per_step": 4 * (w["prompt"] + w["decode"]),
                "d2h_bytes_per_step": 4 * (w["vocab"] // tp) * (w["decode"] + 1),
                "what": "vkl_model_forward per token: host id in, fp32 logits out, host arg-max"},
        "parity": parity,
        "gpu_launches": int(launches), "clocks": clocks, "wall_s": wall,
    }
    if anchor is not None and tp == 1:
        line["tp_anchor"] = anchor
    if f16w:
        # dense prefill on the tensor cores: 2 flops per weight per prompt token (attention and the 1-row lm head left out)
        d, f, nl = w["dim"], w["ffn"], w["layers"]
        flops = 2.0 * w["prompt"] * nl * (4 * d * d + 3 * f * d)
        tf = flops / (float(np.mean(pre_ms)) * 1e-3) / 1e12
        tpeak, tkind = peak_tensor()
        line["roofline_prefill"] = {"bound": "tensor", "what": "whole prefill pass (GEMMs + attention + norms) over projection flops",
                                    "achieved": tf, "peak": tpeak, "unit": "TFLOP/s", "frac": tf / tpeak, "peak_kind": tkind,
                                    "prefill_tokens_per_s": w["prompt"] / (float(np.mean(pre_ms)) * 1e-3)}
    if not args.no_cpu_baseline and world == 1 and not f16w:
        v, cores, sample = cpu_port_tokens_per_s(w)
        line["cpu_baseline"] = {"value": v, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample}
    print(json.dumps(line))
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
