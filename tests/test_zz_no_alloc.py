"""The arg-max entry point that allocates nothing (vkl_argmax_noalloc), called through
the C ABI with raw device pointers, against the ArgMax op on the same inputs.

It exists for callers that cannot allocate device memory where they need the greedy
pick (a serving loop that handed out its memory budget at start-up, code inside a stream
capture): its scratch is a fixed array inside the library that every call shares and that
keeps the previous call's contents, so the check runs two calls in a row with different
inputs. This file is collected last on purpose: a failure here stops nothing else.
"""
import ctypes as C

import numpy as np
import pytest

from oracle import oracle as O
import vkllama_b200 as vk

pytestmark = pytest.mark.gpu


def test_argmax_noalloc_matches_argmax_op_on_two_calls_in_a_row():
    dev = vk.Device(0)
    L = vk.load_library()
    cmd = vk.Command(dev)
    stream = cmd.stream()
    shapes = [(1, 32000), (7, 5000)]  # a vocabulary row, then a ragged multi-row case
    for call, (rows, width) in enumerate(shapes):
        x = O.synth_f16(171, 10 + call, rows * width).reshape(1, rows, width)
        xf = O.f16(x).reshape(rows, width)
        xf[0, [width - 1, 3]] = xf.max() + 1.0  # a tie: the lowest index must win
        x = O.bits(xf).reshape(1, rows, width)
        cmd.begin()
        tx = vk.Tensor(1, rows, width, dev, vk.FP16)
        out = vk.Tensor(1, rows, 1, dev, vk.UINT32)
        cmd.upload(x, tx)
        op = vk.ArgMax(dev, cmd, vk.FP16).init()
        want = cmd.download(op(tx))
        st = L.vkl_argmax_noalloc(tx.device_ptr(), rows, width, out.device_ptr(), stream)
        assert st == 0, L.vkl_last_error()
        got = cmd.download(out)
        cmd.end()
        cmd.submit_and_wait()
        assert np.array_equal(got.ravel(), want.ravel()), "call %d" % call
        assert got.ravel()[0] == 3
        assert np.array_equal(got.ravel(), np.argmax(O.f16(x).reshape(rows, width), 1))
    # sizes beyond the built-in scratch are refused, nothing is launched
    st = L.vkl_argmax_noalloc(tx.device_ptr(), 9000, 1024, out.device_ptr(), stream)
    assert st == 11 and b"8192" in L.vkl_last_error()
    assert L.vkl_argmax_noalloc(None, 1, 8, out.device_ptr(), stream) == 3
    # a pointer that is not memory of the current device is refused on the host, before any launch
    host = np.zeros(64, np.uint16)
    assert L.vkl_argmax_noalloc(host.ctypes.data_as(C.c_void_p), 1, 64, out.device_ptr(), stream) == 3
    dev.close()
