"""Host-side bookkeeping of the persistent decode kernel (tile order of the packed weight stream, stage
cutting, attention split ranges), compiled from csrc/kernels.h with the host compiler and run on the CPU."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_stream_layout_and_stage_cuts(tmp_path):
    cuda_inc = "/usr/local/cuda/include"
    if not shutil.which("g++") or not os.path.isdir(cuda_inc):
        pytest.skip("needs g++ and the CUDA headers")
    exe = str(tmp_path / "test_stream_layout")
    src = os.path.join(ROOT, "tests", "cpp", "test_stream_layout.cpp")
    r = subprocess.run(["g++", "-std=c++17", "-O1", "-I", cuda_inc, "-I", os.path.join(ROOT, "vkllama_b200", "csrc"), src, "-o", exe],
                       capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-3000:]
    r = subprocess.run([exe], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and r.stdout.strip().endswith("OK"), r.stdout[-2000:] + r.stderr[-2000:]
