"""Builds libfaws.so (the C-ABI library of include/faws.h) in-tree with nvcc for sm_100a.

    python -m flash_attn_with_score_b200.build [--force] [--verbose]
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
LIB = os.environ.get("FAWS_LIB_PATH") or os.path.join(HERE, "libfaws.so")
SOURCES = ["faws_abi.cu", "faws_generic.cu", "faws_tc.cu", "faws_noalloc.cu"]
HEADERS = ["faws_internal.cuh", "faws_tc_ptx.cuh"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.sep not in cand or os.path.exists(cand)):
            return cand
    return "nvcc"


def needs_build() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, f) for f in SOURCES + HEADERS] + [os.path.join(ROOT, "include", "faws.h")]
    return any(os.path.exists(d) and os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not needs_build():
        return LIB
    cmd = [
        _nvcc(), "-shared", "-Xcompiler", "-fPIC", "-O3", "-std=c++17", "-lineinfo",
        "-gencode", "arch=compute_100a,code=sm_100a",
        "-I", os.path.join(ROOT, "include"), "-I", CSRC,
        "-o", LIB,
    ] + [os.path.join(CSRC, s) for s in SOURCES] + ["-lcuda"]
    if os.environ.get("FAWS_NVCC_FLAGS"):
        cmd[1:1] = os.environ["FAWS_NVCC_FLAGS"].split()
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed building libfaws.so")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
