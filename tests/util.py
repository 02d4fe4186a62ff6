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
