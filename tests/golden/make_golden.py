"""Generates tests/golden/q8_0_reference.npz with the reference's own quantizer.

Run in the authoring container, where the reference tree is mounted:

    python tests/golden/make_golden.py

It builds oracle/_ref/libref_quants.so from the reference's src/core/quants.{h,cpp}
(recipe: oracle/Makefile), quantizes seeded inputs with it, and stores inputs and
the reference's 36-byte blocks. The committed .npz lets machines without the
reference tree (the GPU box) pin the oracle and the product quantizers.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import oracle as O  # noqa: E402


def main():
    R = O.ref()
    assert R is not None, "oracle/_ref is not built (reference tree missing?)"
    cases = {}
    rng = np.random.default_rng(20240601)
    inputs = {
        "n95": O.synth_f32(11, 1, 3 * 95, 0.0, 1.0).reshape(3, 95),              # tests/test_quants.cpp:21-53 (n = 95)
        "w4096": O.synth_f32(11, 2, 4 * 4096, 0.0, 0.02).reshape(4, 4096),       # N(0, 0.02) weight rows
        "w11008": O.synth_f32(11, 3, 2 * 11008, 0.0, 0.02).reshape(2, 11008),
        "zeros": np.zeros((2, 64), np.float32),                                  # scale 0 -> inverse 0
        "ties": (rng.integers(-254, 255, size=(4, 64)).astype(np.float32) / 2.0),  # x.5 codes: round half away
        "huge": (rng.standard_normal((2, 96)) * 1e4).astype(np.float32),
        "tiny": (rng.standard_normal((2, 40)) * 1e-6).astype(np.float32),
        "one": np.array([[3.25]], np.float32),
    }
    for name, x in inputs.items():
        x = np.ascontiguousarray(x, np.float32)
        h, w = x.shape
        out = np.empty(h * ((w + 31) // 32) * 36, np.int8)
        assert R.ref_q8_0_quantize(x, out, h, w) == 0
        deq = np.empty((h, w), np.float32)
        assert R.ref_q8_0_dequantize(out, deq, h, w) == 0
        cases[name + "_x"] = x
        cases[name + "_q36"] = out.view(np.uint8)
        cases[name + "_deq"] = deq
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "q8_0_reference.npz")
    np.savez_compressed(path, **cases)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
