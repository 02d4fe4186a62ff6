"""GGUF reader and host samplers on the CPU (no device needed): a synthetic checkpoint written
by the `gguf` Python package is read back through the C ABI, and the samplers are compared with
a numpy restatement of models/samplers.cpp:16-101."""
import os

import numpy as np
import pytest

from oracle import oracle as O
import vkllama_b200 as vk

gguf = pytest.importorskip("gguf")

CFG = dict(dim=64, heads=4, ffn=96, vocab=40, layers=2, maxlen=64)


def write_gguf(path, om, cfg, f16=False, extra=None):
    """A checkpoint with the keys and tensor names Model::init reads (models/llama2.h:367-370, 401-512)."""
    w = gguf.GGUFWriter(path, "llama")
    w.add_uint32("llama.attention.head_count", cfg["heads"])
    w.add_uint32("llama.block_count", cfg["layers"])
    w.add_float32("llama.attention.layer_norm_rms_epsilon", 1e-5)
    w.add_uint32("llama.context_length", cfg["maxlen"])
    w.add_uint32("llama.embedding_length", cfg["dim"])
    w.add_array("tokenizer.ggml.tokens", ["<unk>", "<s>", "</s>", "a"])  # a string array the reader must skip over
    w.add_array("tokenizer.ggml.scores", [0.0, -1.0, -2.0, -3.0])
    if extra:
        extra(w)
    from util import llama_names
    L = cfg["layers"]
    tensors = {}

    def add(name, slot_w, rows, cols, norm):
        if norm:
            a = np.ascontiguousarray(slot_w.view(np.float32))
            w.add_tensor(name, a)
        elif f16:
            a = np.ascontiguousarray(slot_w.view(np.uint16).reshape(rows, cols)).view(np.float16)
            w.add_tensor(name, a)
        else:
            a = np.ascontiguousarray(slot_w.view(np.uint8).reshape(rows, cols // 32 * 34))
            w.add_tensor(name, a, raw_dtype=gguf.GGMLQuantizationType.Q8_0)
        tensors[name] = np.ascontiguousarray(slot_w).view(np.uint8).ravel()

    d, f, v = cfg["dim"], cfg["ffn"], cfg["vocab"]
    shapes = dict(attn_norm=(1, d), wq=(d, d), wk=(d, d), wv=(d, d), wo=(d, d), ffn_norm=(1, d), gate=(f, d), up=(f, d), down=(d, f))
    for slot, name in llama_names().items():
        r, c = (1, d) if slot == "output_norm" else (v, d)
        add(name, om.weight(L, O.GLOBALS[slot]), r, c, slot == "output_norm")
    for l in range(L):
        for slot, name in llama_names(l).items():
            add(name, om.weight(l, O.SLOTS[slot]), *shapes[slot], slot.endswith("norm"))
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()
    return tensors


def test_gguf_reader_matches_written_file(tmp_path):
    om = O.Model(seed=21, **CFG)
    path = str(tmp_path / "toy.gguf")
    tensors = write_gguf(path, om, CFG)
    g = vk.Gguf(path)
    version, n_keys, n_tensors = g.counts()
    assert version == 3 and n_tensors == 3 + 9 * CFG["layers"] and n_keys >= 7
    assert g.u32("llama.attention.head_count") == CFG["heads"]
    assert g.u32("llama.block_count") == CFG["layers"]
    assert g.u32("llama.context_length") == CFG["maxlen"]
    assert abs(g.f32("llama.attention.layer_norm_rms_epsilon") - 1e-5) < 1e-12
    assert g.string("general.architecture") == "llama"
    seen = set()
    for i in range(n_tensors):
        t = g.tensor(i)
        seen.add(t["name"])
        assert np.array_equal(t["data"], tensors[t["name"]]), t["name"]
        assert np.array_equal(g.tensor(t["name"])["data"], t["data"])
    assert seen == set(tensors)
    t = g.tensor("blk.1.ffn_down.weight")
    assert t["dims"] == [CFG["ffn"], CFG["dim"]] and t["type"] == 8  # row length first; 8 = Q8_0 (llama2.h:382-397)
    assert g.tensor("output_norm.weight")["type"] == 0
    with pytest.raises(vk.VklError) as e:
        g.u32("llama.rope.dimension_count")
    assert e.value.code == 5
    with pytest.raises(vk.VklError) as e:
        g.tensor("blk.9.attn_q.weight")
    assert e.value.code == 5
    with pytest.raises(vk.VklError) as e:
        g.f32("llama.block_count")  # an integer key read as float
    assert e.value.code == 3
    g.close()


def test_gguf_custom_alignment_and_f16(tmp_path):
    om = O.Model(seed=22, fp16=True, **CFG)
    path = str(tmp_path / "toy16.gguf")
    tensors = write_gguf(path, om, CFG, f16=True, extra=lambda w: w.add_custom_alignment(64))
    g = vk.Gguf(path)
    t = g.tensor("blk.0.attn_q.weight")
    assert t["type"] == 1 and t["dims"] == [CFG["dim"], CFG["dim"]]
    assert np.array_equal(t["data"], tensors["blk.0.attn_q.weight"])
    assert t["data"].ctypes.data % 64 == 0
    g.close()


def test_gguf_rejects_broken_files(tmp_path):
    with pytest.raises(vk.VklError) as e:
        vk.Gguf(str(tmp_path / "missing.gguf"))
    assert e.value.code == 5
    p = tmp_path / "junk.gguf"
    p.write_bytes(b"GGML" + bytes(60))
    with pytest.raises(vk.VklError) as e:
        vk.Gguf(str(p))
    assert e.value.code == 3
    om = O.Model(seed=23, **CFG)
    good = str(tmp_path / "good.gguf")
    write_gguf(good, om, CFG)
    raw = open(good, "rb").read()
    for cut in (30, 200, len(raw) - 100):  # inside the keys, inside the tensor table, inside the data
        q = tmp_path / ("cut%d.gguf" % cut)
        q.write_bytes(raw[:cut])
        with pytest.raises(vk.VklError) as e:
            vk.Gguf(str(q))
        assert e.value.code in (3, 11), cut
    v9 = tmp_path / "v9.gguf"
    v9.write_bytes(raw[:4] + (9).to_bytes(4, "little") + raw[8:])
    with pytest.raises(vk.VklError) as e:
        vk.Gguf(str(v9))
    assert e.value.code == 12


# ---- samplers ------------------------------------------------------------------------------
def ref_topk_probs(logits, k):
    """models/samplers.cpp:37-64: sort descending, keep k, softmax with the first entry as maximum."""
    order = np.lexsort((np.arange(logits.size), -logits))[:k]
    e = np.exp(logits[order] - logits[order[0]], dtype=np.float32)
    return order, e / e.sum(dtype=np.float32)


def ref_topp_set(logits, p):
    """models/samplers.cpp:67-101: shortest sorted prefix whose softmax mass (over all logits) reaches p."""
    order = np.lexsort((np.arange(logits.size), -logits))
    e = np.exp(logits[order] - logits[order[0]], dtype=np.float32)
    pr = e / e.sum(dtype=np.float32)
    acc, keep = np.float32(0), 0
    while keep < logits.size and acc < p:
        acc += pr[keep]
        keep += 1
    kept = order[:keep]
    e2 = np.exp(logits[kept] - logits[kept[0]], dtype=np.float32)
    return kept, e2 / e2.sum(dtype=np.float32)


def test_topk_one_is_argmax_with_lowest_index_on_ties():
    rng = np.random.default_rng(1)
    s = vk.TopkSampler(1, seed=5)
    for _ in range(20):
        x = rng.standard_normal(32000).astype(np.float32)
        assert s.sample(x) == int(np.argmax(x))
    x = np.zeros(100, np.float32)
    x[[17, 40, 99]] = 3.0
    assert s.sample(x) == 17


def test_topk_draws_follow_the_softmax_over_the_k_largest():
    rng = np.random.default_rng(2)
    x = (rng.standard_normal(5000) * 2).astype(np.float32)
    order, pr = ref_topk_probs(x, 8)
    s = vk.TopkSampler(8, seed=11)
    n = 20000
    draws = np.array([s.sample(x) for _ in range(n)])
    assert set(draws.tolist()) <= set(order.tolist())
    freq = np.array([(draws == i).mean() for i in order])
    assert np.abs(freq - pr).max() < 4 * np.sqrt(0.25 / n) + 1e-3, (freq, pr)
    # candidates from a device top-k give the same distribution
    s2 = vk.TopkSampler(8, seed=12)
    d2 = np.array([s2.sample_candidates(x[order], order.astype(np.uint32)) for _ in range(n)])
    f2 = np.array([(d2 == i).mean() for i in order])
    assert np.abs(f2 - pr).max() < 4 * np.sqrt(0.25 / n) + 1e-3
    # k beyond the row length keeps every entry
    s3 = vk.TopkSampler(40, seed=1)
    assert s3.sample(np.array([0.0, 50.0, 1.0], np.float32)) == 1


def test_same_seed_same_draws():
    x = np.linspace(-1, 1, 300).astype(np.float32)
    a, b = vk.TopkSampler(40, seed=99), vk.TopkSampler(40, seed=99)
    assert [a.sample(x) for _ in range(50)] == [b.sample(x) for _ in range(50)]


@pytest.mark.parametrize("p", [0.1, 0.5, 0.9, 1.0])
def test_topp_keeps_the_shortest_prefix_reaching_p(p):
    rng = np.random.default_rng(3)
    x = (rng.standard_normal(2000) * 3).astype(np.float32)
    kept, pr = ref_topp_set(x, p)
    s = vk.TopPSampler(p, seed=21)
    n = 6000
    draws = np.array([s.sample(x) for _ in range(n)])
    assert set(draws.tolist()) <= set(kept.tolist())
    top = kept[:5]
    freq = np.array([(draws == i).mean() for i in top])
    assert np.abs(freq - pr[:5]).max() < 4 * np.sqrt(0.25 / n) + 1e-3
    if kept.size <= 8:
        assert set(draws.tolist()) == set(kept.tolist())


def test_sampler_argument_errors():
    with pytest.raises(vk.VklError) as e:
        vk.TopkSampler(0)
    assert e.value.code == 3
    with pytest.raises(vk.VklError) as e:
        vk.TopPSampler(0.0)
    assert e.value.code == 3
    with pytest.raises(vk.VklError) as e:
        vk.TopPSampler(0.5).sample_candidates(np.ones(3, np.float32), np.arange(3, dtype=np.uint32))
    assert e.value.code == 9
