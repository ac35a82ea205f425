"""The reference-side code compiles and links on its own: the free-function shims (tqllm_b200/adapter/tqllm_shims.cpp)
against include/b2moe.h, and the WeightFormat adapter (tqllm_b200/adapter/b200_expert_format.cpp) against the reference's
own weight_format.hpp where that checkout exists, both with -Wall -Werror and --no-undefined, and the driver program of the
GPU adapter test links the shims through the reference's declarations (moe_kernels.cuh): a signature that differs from the
reference's would be an undefined symbol."""
import os
import shutil
import subprocess

import pytest

import adapter_build

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


@pytest.mark.skipif(shutil.which("g++") is None or not adapter_build.reference_headers(), reason="needs g++ and the reference checkout's headers")
def test_adapter_compiles_against_the_reference_header():
    try:
        driver = adapter_build.build()
    except subprocess.CalledProcessError as e:
        pytest.fail(e.stderr[-3000:])
    assert os.path.isfile(driver) and os.path.isfile(adapter_build.LIB)
