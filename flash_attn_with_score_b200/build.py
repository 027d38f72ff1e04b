"""Builds libfaws.so (the C-ABI library of include/faws.h) in-tree with nvcc for sm_100a.

    python -m flash_attn_with_score_b200.build [--force] [--verbose]

Each translation unit is compiled to an object file under build/ (in parallel, only when the
content of its source or headers changed) and the objects are linked into
flash_attn_with_score_b200/libfaws.so.
"""
from __future__ import annotations

import concurrent.futures
import hashlib
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
OBJDIR = os.path.join(ROOT, "build", "libfaws")
LIB = os.path.join(HERE, "libfaws.so")
SOURCES = ["faws_abi.cu", "faws_generic.cu", "faws_tc.cu", "faws_tc_scores.cu", "faws_bwd.cu", "faws_tc_bwd.cu", "faws_noalloc.cu"]
HEADERS = ["faws_internal.cuh", "faws_tc_ptx.cuh", "faws_tc_host.cuh"]
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.sep not in cand or os.path.exists(cand)):
            return cand
    return "nvcc"


def _deps() -> list[str]:
    return [os.path.join(CSRC, f) for f in HEADERS] + [os.path.join(ROOT, "include", "faws.h")]


def _digest(paths: list[str], extra: str = "") -> str:
    """Content hash of the files an artefact is made from (mtimes lie when files change during a build)."""
    h = hashlib.sha256(extra.encode())
    for path in paths:
        h.update(path.encode())
        if os.path.exists(path):
            with open(path, "rb") as f:
                h.update(f.read())
    return h.hexdigest()


def _read(path: str) -> str:
    try:
        with open(path) as f:
            return f.read().strip()
    except OSError:
        return ""


def _lib_digest() -> str:
    return _digest([os.path.join(CSRC, f) for f in SOURCES] + _deps(), " ".join(ARCH))


def needs_build() -> bool:
    return not os.path.exists(LIB) or _read(os.path.join(OBJDIR, "libfaws.digest")) != _lib_digest()


def _compile(src: str, force: bool, verbose: bool) -> tuple[str, int, str]:
    obj = os.path.join(OBJDIR, os.path.splitext(src)[0] + ".o")
    path = os.path.join(CSRC, src)
    digest = _digest([path] + _deps(), " ".join(ARCH))
    if not force and os.path.exists(obj) and _read(obj + ".digest") == digest:
        return obj, 0, ""
    cmd = [_nvcc(), "-c", "-Xcompiler", "-fPIC", "-O3", "-std=c++17", "-lineinfo"] + ARCH + [
        "-I", os.path.join(ROOT, "include"), "-I", CSRC, "-o", obj, path]
    if verbose:
        cmd[1:1] = ["-Xptxas", "-v"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode == 0:
        with open(obj + ".digest", "w") as f:
            f.write(digest)  # the digest of what was read before the compile started
    return obj, res.returncode, res.stdout + res.stderr


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not needs_build():
        return LIB
    os.makedirs(OBJDIR, exist_ok=True)
    lib_digest = _lib_digest()
    with concurrent.futures.ThreadPoolExecutor(max_workers=len(SOURCES)) as pool:
        results = list(pool.map(lambda s: _compile(s, force, verbose), SOURCES))
    failed = False
    for obj, rc, log in results:
        if verbose or rc != 0:
            sys.stderr.write(log)
        failed = failed or rc != 0
    if failed:
        raise RuntimeError("nvcc failed building libfaws.so")
    cmd = [_nvcc(), "-shared"] + ARCH + ["-o", LIB] + [obj for obj, _, _ in results] + ["-lcuda"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed linking libfaws.so")
    if lib_digest == _lib_digest():  # nothing changed while compiling
        with open(os.path.join(OBJDIR, "libfaws.digest"), "w") as f:
            f.write(lib_digest)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
