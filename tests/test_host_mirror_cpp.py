"""The C++ host mirror (include/ullm_cuda.hpp, the stand-in for the `ullm-cuda` crate where the host is compiled
code) builds with plain g++ against the C ABI and behaves like the reference wrapper on a machine without a
GPU: probes answer, connect() refuses, nothing falls back to the CPU."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB_DIR = os.path.join(ROOT, "ullm-project_b200", "lib")


def build(tmp_path):
    exe = str(tmp_path / "host_mirror_test")
    cmd = ["g++", "-std=c++17", "-Wall", "-Wextra", "-Werror", "-O1", "-I" + os.path.join(ROOT, "include"),
           os.path.join(ROOT, "tests", "cpp", "host_mirror_test.cpp"), "-o", exe, "-L" + LIB_DIR, "-lullm_cuda",
           "-Wl,-rpath," + LIB_DIR]
    env = {k: v for k, v in os.environ.items() if k not in ("CC", "CXX")}
    subprocess.run(cmd, check=True, env=env)
    return exe


@pytest.mark.skipif(shutil.which("g++") is None, reason="g++ not on PATH")
def test_cpp_host_mirror_without_a_gpu(tmp_path):
    import torch

    if torch.cuda.is_available():
        pytest.skip("covered by the GPU variant")
    out = subprocess.run([build(tmp_path), "0"], capture_output=True, text=True)
    assert out.returncode == 0, out.stderr
    assert "host mirror ok" in out.stdout


@pytest.mark.gpu
@pytest.mark.skipif(shutil.which("g++") is None, reason="g++ not on PATH")
def test_cpp_host_mirror_with_a_gpu(tmp_path):
    out = subprocess.run([build(tmp_path), "1"], capture_output=True, text=True)
    assert out.returncode == 0, out.stderr
    assert "host mirror ok" in out.stdout
