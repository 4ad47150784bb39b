"""The C++ mirror of the reference's Backend interface (include/tpb200.hpp).

CPU: the header and its test program compile (g++, CUDA runtime headers only).
GPU: the test program runs: ConvRot linears and the GGUF GEMVs through tpb::Backend,
compared with the CPU checker inside the program (tests/cpp/test_backend.cpp)."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = os.path.join(ROOT, "tests", "cpp", "test_backend.cpp")
CUDA_INC = "/usr/local/cuda/include"
CUDA_LIB = "/usr/local/cuda/lib64"


def _compile(out):
    from oracle import oracle
    from tensorpencil_b200 import build
    oracle.build()
    build.build(verbose=False)
    gxx = shutil.which("g++")
    if gxx is None or not os.path.isdir(CUDA_INC):
        pytest.skip("no g++ / CUDA headers")
    lib_dir = os.path.join(ROOT, "tensorpencil_b200", "lib")
    ora_dir = os.path.join(ROOT, "oracle")
    cmd = [gxx, "-std=c++17", "-O1", "-Wall", "-I", os.path.join(ROOT, "include"), "-I", ora_dir, "-I", CUDA_INC,
           SRC, "-o", out, "-L", lib_dir, "-ltpb200", "-L", ora_dir, "-ltpb_oracle", "-L", CUDA_LIB, "-lcudart",
           f"-Wl,-rpath,{lib_dir}", f"-Wl,-rpath,{ora_dir}", f"-Wl,-rpath,{CUDA_LIB}"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-4000:]


def test_cpp_mirror_compiles(tmp_path):
    _compile(str(tmp_path / "test_backend"))


@pytest.mark.gpu
def test_cpp_mirror_runs(tmp_path):
    exe = str(tmp_path / "test_backend")
    _compile(exe)
    r = subprocess.run([exe], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and r.stdout.strip().endswith("OK"), r.stdout[-4000:] + r.stderr[-2000:]
