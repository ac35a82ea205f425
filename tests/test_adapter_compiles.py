"""The reference-side shims (tqllm_b200/adapter/tqllm_shims.cpp: tqLLM's free functions of the expert path written against
include/b2moe.h) compile as plain C++ against the header and link against the built library with no undefined symbol:
the argument lists of the C ABI are what a tqLLM build would bind."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = os.path.join(ROOT, "tqllm_b200", "adapter", "tqllm_shims.cpp")
CUDA_INC = "/usr/local/cuda/include"


@pytest.mark.skipif(shutil.which("g++") is None or not os.path.isdir(CUDA_INC), reason="needs g++ and the CUDA headers")
def test_shims_compile_and_link(tmp_path):
    lib = os.path.join(ROOT, "tqllm_b200", "libb2moe.so")
    assert os.path.isfile(lib), "build the library first (python -m tqllm_b200.build)"
    out = str(tmp_path / "libshims.so")
    cmd = ["g++", "-std=c++17", "-shared", "-fPIC", "-Wall", "-Werror", "-I" + os.path.join(ROOT, "include"), "-I" + CUDA_INC, SRC,
           "-o", out, "-Wl,--no-undefined", lib, "-L/usr/local/cuda/lib64", "-lcudart"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
