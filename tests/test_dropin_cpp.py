"""The static archive as a drop-in for the original libcutt.a: a C++ program that only knows
the original header is compiled with g++ and linked with -lcutt -lcudart (the original link
line, Makefile:105,115-128 of the reference), then run on the GPU."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = os.path.join(ROOT, "tests", "cpp", "dropin_example.cpp")
CUDA = os.environ.get("CUDA_HOME", "/usr/local/cuda")


def _build(native, tmpdir):
    exe = os.path.join(str(tmpdir), "dropin_example")
    libdir = os.path.dirname(native.lib_path())
    cmd = ["g++", "-std=c++11", "-O1", SRC, "-I", os.path.join(ROOT, "include"), "-I", os.path.join(CUDA, "include"),
           "-L", libdir, "-l:libcutt.a", "-L", os.path.join(CUDA, "lib64"), "-lcudart", "-lstdc++", "-lpthread", "-ldl",
           "-o", exe]
    res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    assert res.returncode == 0, res.stdout
    return exe


@pytest.mark.skipif(shutil.which("g++") is None or not os.path.exists(os.path.join(CUDA, "lib64")),
                    reason="needs g++ and the CUDA runtime library")
def test_links_with_cudart_only(native, tmp_path):
    exe = _build(native, tmp_path)
    assert os.path.exists(exe)


@pytest.mark.gpu
def test_runs_bit_exact(native, tmp_path):
    exe = _build(native, tmp_path)
    env = dict(os.environ)
    env["LD_LIBRARY_PATH"] = os.path.join(CUDA, "lib64") + ":" + env.get("LD_LIBRARY_PATH", "")
    res = subprocess.run([exe], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, env=env, timeout=300)
    assert res.returncode == 0, res.stdout
    assert "drop-in example ok" in res.stdout
