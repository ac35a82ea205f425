"""Builds the CPU checker libraries. TEST INFRASTRUCTURE ONLY.

  oracle/_build/liboracle.so  from oracle/oracle.cpp (the restatement; always built)
  oracle/_ref/libtqref.so     from the reference's own sources compiled where they lie in the reference checkout
                              (src/experts/moe.cpp, src/formats/weight/dequant.cpp) plus oracle/ref_shim.cpp; built only
                              when that checkout is present. No reference source is copied into this tree.
  oracle/_ref/libtqrefpool.so the reference's production CPU expert pool (CpuMissPool, a header:
                              src/models/qwen/qwen4exp/fn_cpu_experts.hpp) + dequant.cpp + oracle/ref_pool_shim.cpp: the CPU
                              arm the benchmark times (x86 with AVX2 only).

The checkout is found through the environment variable TQLLM_REFERENCE (a directory holding src/experts/moe.cpp).

Usage: python oracle/build.py [--force]
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
REF = os.environ.get("TQLLM_REFERENCE") or os.path.join(os.path.dirname(ROOT), "reference")   # sibling checkout unless told otherwise
ORACLE_SO = os.path.join(HERE, "_build", "liboracle.so")
REF_SO = os.path.join(HERE, "_ref", "libtqref.so")
POOL_SO = os.path.join(HERE, "_ref", "libtqrefpool.so")
CXXFLAGS = ["-O2", "-std=c++20", "-shared", "-fPIC", "-pthread", "-mavx2", "-mfma", "-mf16c"]


def _stale(out: str, srcs: list[str]) -> bool:
    if not os.path.isfile(out):
        return True
    t = os.path.getmtime(out)
    return any(os.path.getmtime(s) > t for s in srcs if os.path.isfile(s))


def _run(cmd: list[str]) -> None:
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode:
        raise RuntimeError("build failed: " + " ".join(cmd) + "\n" + r.stdout + r.stderr)


def build_oracle(force: bool = False) -> str:
    sys.path.insert(0, ROOT)
    from tqllm_b200 import gen_tables
    tables = gen_tables.write()
    src = os.path.join(HERE, "oracle.cpp")
    if force or _stale(ORACLE_SO, [src, tables]):
        os.makedirs(os.path.dirname(ORACLE_SO), exist_ok=True)
        _run(["g++", *CXXFLAGS, src, "-o", ORACLE_SO])
    return ORACLE_SO


def reference_present() -> bool:
    return os.path.isfile(os.path.join(REF, "src", "experts", "moe.cpp"))


def build_ref(force: bool = False) -> str | None:
    """The reference's CPU path, compiled from its own files in place. Returns None when there is no checkout."""
    if not reference_present():
        return REF_SO if os.path.isfile(REF_SO) else None
    srcs = [os.path.join(REF, "src", "experts", "moe.cpp"), os.path.join(REF, "src", "formats", "weight", "dequant.cpp"),
            os.path.join(HERE, "ref_shim.cpp")]
    if force or _stale(REF_SO, srcs):
        os.makedirs(os.path.dirname(REF_SO), exist_ok=True)
        inc = [f"-I{os.path.join(REF, 'src', d)}" for d in ("experts", "formats/weight", "core")]
        inc += [f"-I{os.path.join(REF, 'include')}", "-I/usr/local/cuda/include"]
        _run(["g++", *CXXFLAGS, *inc, *srcs, "-o", REF_SO])
    return REF_SO


def build_ref_pool(force: bool = False) -> str | None:
    """The reference's production CPU expert pool, compiled from its own header in place. None when it cannot be had."""
    if not reference_present():
        return POOL_SO if os.path.isfile(POOL_SO) else None
    hdr = os.path.join(REF, "src", "models", "qwen", "qwen4exp", "fn_cpu_experts.hpp")
    srcs = [os.path.join(REF, "src", "formats", "weight", "dequant.cpp"), os.path.join(HERE, "ref_pool_shim.cpp")]
    if force or _stale(POOL_SO, srcs + [hdr]):
        os.makedirs(os.path.dirname(POOL_SO), exist_ok=True)
        inc = []
        for d, _, _ in os.walk(os.path.join(REF, "src")):
            inc.append(f"-I{d}")
        inc += [f"-I{os.path.join(REF, 'include')}", f"-I{os.path.join(REF, 'third_party')}", "-I/usr/local/cuda/include"]
        try:
            _run(["g++", *CXXFLAGS, *inc, *srcs, "-o", POOL_SO])
        except RuntimeError:
            return None          # not an x86 / AVX2 host, or a checkout without the pool
    return POOL_SO


if __name__ == "__main__":
    force = "--force" in sys.argv
    print(build_oracle(force))
    print(build_ref(force))
    print(build_ref_pool(force))
