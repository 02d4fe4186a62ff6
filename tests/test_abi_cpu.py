"""The C-ABI library loads without a GPU, exports every symbol the header
declares, and reports errors as status codes (no compute calls here)."""
import ctypes as C
import os
import re

import numpy as np
import pytest

import vkllama_b200 as vk

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "vkllama_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(vkl_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    L = vk.load_library()
    names = declared_symbols()
    assert len(names) >= 60
    for n in names:
        assert hasattr(L, n), "missing export: " + n


def _has_gpu():
    try:
        vk.Device(0).close()
        return True
    except vk.VklError:
        return False


def test_device_create_fails_loudly_without_a_gpu():
    if _has_gpu():
        pytest.skip("a CUDA device is present")
    with pytest.raises(vk.VklError) as e:
        vk.Device(0)
    assert e.value.code == 9  # FAILED_PRECONDITION
    assert "no CPU fallback" in e.value.message


def test_null_and_bad_arguments_return_status_codes():
    L = vk.load_library()
    assert L.vkl_device_create(0, None) == 3
    assert L.vkl_tensor_create(None, 1, 1, 1, vk.FP16, C.byref(C.c_void_p())) == 3
    assert L.vkl_command_begin(None) == 3
    assert L.vkl_op_init(None) == 3
    assert L.vkl_model_forward(None, None, 0, 0, None) == 3
    assert L.vkl_q8_0_quantize(None, None, 1, 1) == 3
    assert b"null" in L.vkl_last_error()
    assert L.vkl_tensor_release(None) == 0 and L.vkl_op_destroy(None) == 0


def test_status_codes_match_absl():
    text = open(os.path.join(ROOT, "include", "vkllama_b200.h")).read()
    for name, val in [("VKL_INVALID_ARGUMENT", 3), ("VKL_OUT_OF_RANGE", 11), ("VKL_UNIMPLEMENTED", 12), ("VKL_INTERNAL", 13)]:
        assert re.search(r"%s\s*=\s*%d\b" % (name, val), text)
    for name, val in [("VKL_FP32", 0), ("VKL_FP16", 1), ("VKL_UINT32", 2), ("VKL_INT8", 3), ("VKL_Q8_0", 4)]:
        assert re.search(r"%s\s*=\s*%d\b" % (name, val), text)  # src/core/common.h:15-22
