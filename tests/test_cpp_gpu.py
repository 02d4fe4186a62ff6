"""Builds and runs the C++ parity program that goes through the header-only class layer
(include/vkllama/vkllama.h -> C ABI), against the CPU oracle."""
import os
import subprocess

import pytest

from oracle import oracle as O

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BIN = os.path.join(ROOT, "tests", "cpp", "test_ops")


def build_cpp_test():
    O.build()
    src = os.path.join(ROOT, "tests", "cpp", "test_ops.cpp")
    cmd = ["/usr/bin/g++", "-std=c++17", "-O2", "-mf16c", "-I", os.path.join(ROOT, "include"), src, "-o", BIN,
           "-L", os.path.join(ROOT, "vkllama_b200"), "-lvkllama_b200", "-L", os.path.join(ROOT, "oracle"), "-loracle",
           "-Wl,-rpath," + os.path.join(ROOT, "vkllama_b200"), "-Wl,-rpath," + os.path.join(ROOT, "oracle")]
    subprocess.check_call(cmd)


def test_cpp_layer_compiles_and_links():
    """No GPU needed: the header-only classes compile against the C ABI and link."""
    build_cpp_test()
    assert os.path.exists(BIN)


@pytest.mark.gpu
def test_cpp_class_layer_parity():
    build_cpp_test()
    r = subprocess.run([BIN], capture_output=True, text=True, timeout=280)
    assert r.returncode == 0 and "PASS" in r.stdout, r.stdout + r.stderr
