"""Seeded synthetic token ids (stand-ins for a tokenised prompt; no dataset is read).

The same counter-based generator as the library's device-side weight generator
(vkl_model_synth_weights) and the CPU oracle use: splitmix64 finaliser over
(seed, tensor id, element index). Pure integer arithmetic, so the ids are the
same on every machine.
"""
import numpy as np

_M = (1 << 64) - 1


def _mix64(z):
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _M
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _M
    return z ^ (z >> 31)


def _key(seed, tensor):
    return _mix64((seed * 0x9E3779B97F4A7C15 + tensor * 0xD1B54A32D192ED03 + 0x2545F4914F6CDD1D) & _M)


def synth_tokens(seed, tensor, n, vocab):
    """n token ids, uniform on [0, vocab), as a uint32 array."""
    key = _key(seed, tensor)
    return np.array([(_mix64((key + (i + 1) * 0x9E3779B97F4A7C15) & _M) >> 11) % vocab for i in range(n)], np.uint32)
