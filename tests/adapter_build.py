"""Builds the adapter check artefacts against the reference's own headers (weight_format.hpp, moe_kernels.cuh), which are
used where they lie in the reference checkout: nothing of the reference is copied.

  tests/_build/libadapter.so     tqllm_b200/adapter/*.cpp + test stubs of the base class, linked with --no-undefined
  tests/_build/adapter_driver    the driver program of tests/test_gpu_adapter.py (finds libb2moe.so through its rpath)

Returns None when the checkout is absent (a prebuilt driver, carried with the tree, is still used by the GPU test)."""
import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
REF = os.environ.get("TQLLM_REFERENCE") or os.path.join(os.path.dirname(ROOT), "reference")
OUT = os.path.join(HERE, "_build")
LIB, DRIVER = os.path.join(OUT, "libadapter.so"), os.path.join(OUT, "adapter_driver")
CUDA = "/usr/local/cuda"


def reference_headers():
    return os.path.isfile(os.path.join(REF, "src", "formats", "weight", "weight_format.hpp")) and os.path.isdir(os.path.join(CUDA, "include"))


def build():
    if not reference_headers():
        return None
    os.makedirs(OUT, exist_ok=True)
    ad = os.path.join(ROOT, "tqllm_b200", "adapter")
    srcs = [os.path.join(ad, "b200_expert_format.cpp"), os.path.join(ad, "tqllm_shims.cpp"), os.path.join(HERE, "adapter_base_stubs.cpp")]
    inc = ["-I" + os.path.join(ROOT, "include"), "-I" + ad, "-I" + os.path.join(REF, "src", "formats", "weight"), "-I" + os.path.join(REF, "src", "experts"),
           "-I" + os.path.join(CUDA, "include")]
    lib = os.path.join(ROOT, "tqllm_b200", "libb2moe.so")
    link = ["-Wl,--no-undefined", lib, "-L" + os.path.join(CUDA, "lib64"), "-lcudart"]
    common = ["g++", "-std=c++20", "-O1", "-fPIC", "-Wall", "-Werror", *inc]
    subprocess.run([*common, "-shared", *srcs, "-o", LIB, *link], check=True, capture_output=True, text=True)
    subprocess.run([*common, *srcs, os.path.join(HERE, "adapter_driver.cpp"), "-o", DRIVER, *link,
                    "-Wl,-rpath,$ORIGIN/../../tqllm_b200", "-Wl,-rpath," + os.path.join(CUDA, "lib64")], check=True, capture_output=True, text=True)
    return DRIVER


if __name__ == "__main__":
    print(build())
