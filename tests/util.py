"""Shared helpers of the parity tests."""
import numpy as np

from oracle import oracle as O
import vkllama_b200 as vk

# Tolerances of the parity contract: per-op fp16 outputs within max-rel 1e-2,
# final logits within max-abs 5e-2, Q8_0 codes and scales bit-exact.
OP_MAX_REL = 1e-2
LOGITS_MAX_ABS = 5e-2


def max_rel(a_bits, b_bits):
    """max |a-b| / max |b| over fp16 bit patterns (b = oracle)."""
    a, b = O.f16(np.asarray(a_bits).ravel()), O.f16(np.asarray(b_bits).ravel())
    assert a.shape == b.shape
    return float(np.abs(a - b).max() / max(np.abs(b).max(), 1e-30))


def assert_close(a_bits, b_bits, tol=OP_MAX_REL, what=""):
    r = max_rel(a_bits, b_bits)
    assert r <= tol, "%s max-rel %.3e > %.1e" % (what, r, tol)
    return r


def up(cmd, dev, arr, dtype, c, h, w):
    t = vk.Tensor(c, h, w, dev, dtype)
    cmd.upload(arr, t)
    return t


def llama_names(layer=None):
    if layer is None:
        return {"tok_embd": "token_embd.weight", "output_norm": "output_norm.weight", "output": "output.weight"}
    m = dict(attn_norm="attn_norm", wq="attn_q", wk="attn_k", wv="attn_v", wo="attn_output",
             ffn_norm="ffn_norm", gate="ffn_gate", up="ffn_up", down="ffn_down")
    return {k: "blk.%d.%s.weight" % (layer, v) for k, v in m.items()}


def load_from_oracle(model, om):
    """Upload every weight of an oracle model into a device model (raw GGUF bytes)."""
    L = om.cfg["layers"]
    wdt = vk.FP16 if getattr(om, "fp16", False) else vk.Q8_0
    for l in range(L):
        for slot, name in llama_names(l).items():
            w = om.weight(l, O.SLOTS[slot])
            if slot.endswith("norm"):
                model.set_weight(name, vk.FP32, w.view(np.float32))
            else:
                model.set_weight(name, wdt, w)
    for slot, name in llama_names().items():
        w = om.weight(L, O.GLOBALS[slot])
        if slot == "output_norm":
            model.set_weight(name, vk.FP32, w.view(np.float32))
        else:
            model.set_weight(name, wdt, w)


def fp16_ulp(v):
    """One fp16 ulp at |v|."""
    return 2.0 ** (np.floor(np.log2(max(abs(float(v)), 2.0 ** -14))) - 10)


def oracle_walk(om, prompt, n_gen):
    """Greedy ids of the oracle and, per step, its top-2 logit gap in fp16 ulps of the top logit."""
    ids, ulps = [], []
    logits = om.forward(np.ascontiguousarray(prompt, np.uint32), 0)
    for i in range(n_gen):
        if i:
            logits = om.forward(np.array([ids[-1]], np.uint32), len(prompt) + i - 1)
        top = int(np.flatnonzero(logits == logits.max())[0])
        second = float(np.max(np.delete(logits, top)))
        ids.append(top)
        ulps.append((float(logits[top]) - second) / fp16_ulp(logits[top]))
    return np.array(ids, np.uint32), np.array(ulps)


def decided_prompt(make_oracle, seed, P, n_gen, vocab, min_ulps=4.0, tries=60):
    """A seeded prompt whose every greedy step the oracle decides by at least `min_ulps` fp16 ulps, so
    that a correct implementation with another fp32 summation order must produce the same ids.
    make_oracle() returns a fresh oracle model (the walk fills its caches). Returns (prompt, ids)."""
    for k in range(tries):
        om = make_oracle()
        prompt = O.synth_tokens(seed, 1000 + k, P, vocab)
        ids, ulps = oracle_walk(om, prompt, n_gen)
        if ulps.min() >= min_ulps:
            return prompt, ids
    raise AssertionError("no prompt with every step decided by %.1f ulps in %d tries" % (min_ulps, tries))
