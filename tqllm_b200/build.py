"""Compiles the CUDA sources of this package for sm_100a into tqllm_b200/libb2moe.so (in-tree, so the built library
travels with the source tree). nvcc cross-compiles without a GPU. Usage: python -m tqllm_b200.build [--force] [-v]"""
from __future__ import annotations

import concurrent.futures as cf
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "_obj")
LIB = os.path.join(HERE, "libb2moe.so")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = ["-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-Xcompiler", "-fPIC",
         "--expt-relaxed-constexpr", "-Xcompiler", "-fvisibility=hidden"]


def sources() -> list[str]:
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def _deps() -> list[str]:
    hdrs = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    hdrs.append(os.path.join(CSRC, "_gen", "ggml_tables.h"))
    hdrs.append(os.path.join(os.path.dirname(HERE), "include", "b2moe.h"))
    return hdrs


def _compile(src: str, verbose: bool) -> str:
    obj = os.path.join(OBJ, os.path.basename(src)[:-3] + ".o")
    cmd = [NVCC, *FLAGS, *(["-Xptxas", "-v"] if verbose else []), "-c", src, "-o", obj]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode:
        raise RuntimeError(f"nvcc failed on {src}:\n{r.stdout}{r.stderr}")
    if verbose:
        sys.stderr.write(r.stderr)
    return obj


def build(force: bool = False, verbose: bool = False) -> str:
    from . import gen_tables
    gen_tables.write()
    os.makedirs(OBJ, exist_ok=True)
    srcs, deps = sources(), _deps()
    newest_hdr = max(os.path.getmtime(d) for d in deps if os.path.isfile(d))
    todo = []
    for s in srcs:
        obj = os.path.join(OBJ, os.path.basename(s)[:-3] + ".o")
        if force or not os.path.isfile(obj) or os.path.getmtime(obj) < max(os.path.getmtime(s), newest_hdr):
            todo.append(s)
    with cf.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as ex:
        list(ex.map(lambda s: _compile(s, verbose), todo))
    objs = [os.path.join(OBJ, os.path.basename(s)[:-3] + ".o") for s in srcs]
    if todo or not os.path.isfile(LIB):
        r = subprocess.run([NVCC, "-shared", "-o", LIB, *objs, "-gencode", "arch=compute_100a,code=sm_100a", "-lcudart"],
                           capture_output=True, text=True)
        if r.returncode:
            raise RuntimeError(f"link failed:\n{r.stdout}{r.stderr}")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
