"""Builds the CPU checker libraries. TEST INFRASTRUCTURE ONLY.

  oracle/_build/liboracle.so  from oracle/oracle.cpp (the restatement; always built)
  oracle/_ref/libtqref.so     from the reference's own sources compiled where they lie in the reference checkout
                              (src/experts/moe.cpp, src/formats/weight/dequant.cpp) plus oracle/ref_shim.cpp; built only
                              when that checkout is present. No reference source is copied into this tree.

Usage: python oracle/build.py [--force]
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
REF = os.environ.get("TQLLM_REFERENCE", "/root/reference")
ORACLE_SO = os.path.join(HERE, "_build", "liboracle.so")
REF_SO = os.path.join(HERE, "_ref", "libtqref.so")
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


if __name__ == "__main__":
    force = "--force" in sys.argv
    print(build_oracle(force))
    print(build_ref(force))
