"""CPU-only checks: the oracle and the product's host quantizer against the
reference's own quantizer (golden vectors made by tests/golden/make_golden.py,
and the live oracle/_ref build when the reference tree is present)."""
import os

import numpy as np
import pytest

from oracle import oracle as O
import vkllama_b200 as vk

GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "q8_0_reference.npz"))
CASES = sorted(k[:-2] for k in GOLD.files if k.endswith("_x"))


@pytest.mark.parametrize("case", CASES)
def test_oracle_quantizer_matches_reference_golden(case):
    x, want = GOLD[case + "_x"], GOLD[case + "_q36"]
    got = O.quantize36(x)
    assert np.array_equal(got, want), case


@pytest.mark.parametrize("case", CASES)
def test_product_host_quantizer_matches_reference_golden(case):
    x, want = GOLD[case + "_x"], GOLD[case + "_q36"]
    assert np.array_equal(vk.q8_0_quantize36(x), want), case
    # 34-byte layout: same codes, scale = fp16(fp32 scale) rounded to nearest even
    b34 = vk.q8_0_quantize(x).reshape(-1, 34)
    b36 = want.reshape(-1, 36)
    assert np.array_equal(b34[:, 2:], b36[:, 4:])
    scale32 = b36[:, :4].copy().view(np.float32).ravel()
    assert np.array_equal(b34[:, :2].copy().view(np.uint16).ravel(), scale32.astype(np.float16).view(np.uint16))
    assert np.array_equal(vk.blocks36_to_34(want), b34.ravel())
    assert np.array_equal(O.quantize34(x), b34.ravel())


@pytest.mark.parametrize("case", CASES)
def test_dequantize_round_trip(case):
    x = GOLD[case + "_x"]
    h, w = x.shape
    if case == "tiny":
        pytest.skip("scales below the fp16 subnormal range flush to 0 in the 34-byte layout")
    deq =vk.q8_0_dequantize(vk.q8_0_quantize(x), h, w)
    # tests/test_quants.cpp:21-53: quantize -> dequantize stays within the block step
    amax = np.abs(x).max()
    assert np.abs(deq - x).max() <= amax / 127.0 * 0.51 + amax * 2e-3 + 1e-30


def test_live_reference_quantizer_if_present():
    R = O.ref()
    if R is None:
        pytest.skip("oracle/_ref not built on this machine")
    assert R.ref_q8_0_bytes_per_block() == 36
    x = O.synth_f32(77, 5, 16 * 4096, 0.0, 0.02).reshape(16, 4096)
    out = np.empty(16 * 128 * 36, np.int8)
    assert R.ref_q8_0_quantize(x, out, 16, 4096) == 0
    assert np.array_equal(out.view(np.uint8), O.quantize36(x))
    assert np.array_equal(out.view(np.uint8), vk.q8_0_quantize36(x))


def test_synth_generator_statistics_and_determinism():
    a = O.synth_f32(1, 2, 1 << 16, 0.0, 0.02)
    b = O.synth_f32(1, 2, 1 << 16, 0.0, 0.02)
    assert np.array_equal(a, b)
    assert abs(a.mean()) < 5e-4 and abs(a.std() - 0.02) < 5e-4
    # windows of one stream agree with the whole
    c = O.synth_f32(1, 2, 100, 0.0, 0.02, first=1000)
    assert np.array_equal(c, a[1000:1100])
    t = O.synth_tokens(3, 1, 1000, 32000)
    assert t.max() < 32000 and len(np.unique(t)) > 900


def test_oracle_matmul_against_numpy():
    N, K = 48, 256
    w = O.synth_q8_0(5, 1, N, K)
    x = O.synth_f16(5, 2, 3 * K).reshape(3, K)
    y = O.matmul_q8_0(x, w, 3, N, K)
    wf = vk.q8_0_dequantize(w, N, K)
    ref = O.f16(x) @ wf.T
    assert np.abs(O.f16(y) - ref).max() <= 2e-3 * np.abs(ref).max() + 1e-3


def test_oracle_softmax_mask_and_argmax_ties():
    L = O.lib()
    x = O.bits(np.array([[1.0, 3.0, 3.0, 2.0]], np.float32))
    out = np.empty(1, np.uint32)
    L.orc_argmax_f16(x, out, 1, 4)
    assert out[0] == 1  # lowest index wins the tie
    s = O.bits(np.zeros((1, 2, 4), np.float32))
    p = np.empty_like(s)
    L.orc_softmax_f16(s, p, 1, 2, 4, 1, 2)  # offset = W - H
    pf = O.f16(p).reshape(2, 4)
    assert np.allclose(pf[0], [1 / 3, 1 / 3, 1 / 3, 0], atol=1e-3)
    assert np.allclose(pf[1], [0.25] * 4, atol=1e-3)


def test_oracle_generate_is_self_consistent():
    m = O.Model(dim=128, heads=4, ffn=256, vocab=320, layers=2, maxlen=64, seed=9)
    prompt = O.synth_tokens(9, 1000, 5, 320)
    ids, gap = m.generate(prompt, 6)
    m2 = O.Model(dim=128, heads=4, ffn=256, vocab=320, layers=2, maxlen=64, seed=9)
    logits = m2.forward(prompt, 0)
    assert int(np.argmax(logits)) == ids[0]
    assert gap[0] >= 0


def test_oracle_fp16_feed_forward_against_numpy():
    M, dim, hidden = 3, 128, 192
    gate = O.synth_f16(31, 1, hidden * dim, 0.0, 0.05)
    down = O.synth_f16(31, 2, dim * hidden, 0.0, 0.05)
    upw = O.synth_f16(31, 3, hidden * dim, 0.0, 0.05)
    x = O.synth_f16(31, 4, M * dim)
    got = np.empty(M * dim, np.uint16)
    O.lib().orc_feed_forward_f16(x, gate, down, upw, got, M, dim, hidden)
    xf = O.f16(x).reshape(M, dim).astype(np.float64)
    g = xf @ O.f16(gate).reshape(hidden, dim).astype(np.float64).T
    u = xf @ O.f16(upw).reshape(hidden, dim).astype(np.float64).T
    t = O.f16(O.bits(g / (1 + np.exp(-g)) * u)).astype(np.float64)
    want = t @ O.f16(down).reshape(dim, hidden).astype(np.float64).T
    err = np.abs(O.f16(got).reshape(M, dim) - want).max() / np.abs(want).max()
    assert err < 2e-3


def test_oracle_fp16_weights_model_runs_and_differs_from_q8_0():
    cfg = dict(dim=128, heads=4, ffn=256, vocab=320, layers=2, maxlen=64, seed=9)
    prompt = O.synth_tokens(9, 1000, 5, 320)
    a = O.Model(fp16=True, **cfg).forward(prompt, 0)
    b = O.Model(fp16=True, **cfg).forward(prompt, 0)
    q = O.Model(**cfg).forward(prompt, 0)
    assert np.isfinite(a).all() and np.array_equal(a, b)
    assert not np.array_equal(a, q) and np.abs(a - q).max() < 0.5  # quantisation noise only
    w = O.Model(fp16=True, **cfg).weight(0, O.SLOTS["wq"])
    assert w.size == 128 * 128 * 2
