"""Builds libginn_b200.so (sm_100a only) in-tree with nvcc.

Usage: python -m ginn_b200.build [--force] [--verbose]
The shared library is the whole product: the Python package and the C++ headers are thin
layers over its C ABI (include/ginn_b200.h).
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libginn_b200.so")
SOURCES = ["api.cu", "grouped_static.cu", "hgemm_tma.cu", "hgemm_pair.cu", "hgemm_gather.cu", "sgemm3x_tma.cu", "small.cu", "step_ops.cu", "conv.cu", "attention.cu"]
HEADERS = ["ptx.cuh", "math.cuh", "problem.h", "launch.h", os.path.join("..", "..", "include", "ginn_b200.h")]


def nvcc_path() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; set NVCC or install the CUDA toolkit")


def stale() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, s) for s in SOURCES + HEADERS] + [os.path.abspath(__file__)]
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not stale():
        return LIB
    from concurrent.futures import ThreadPoolExecutor

    objdir = os.path.join(HERE, "build")
    os.makedirs(objdir, exist_ok=True)
    common = [
        nvcc_path(),
        "-gencode", "arch=compute_100a,code=sm_100a",
        "-lineinfo", "-O3", "-std=c++17",
        "-Xcompiler", "-fPIC,-Wall,-Wno-unused-function",
    ]
    if verbose:
        common += ["-Xptxas", "-v"]

    def compile_one(src: str):
        obj = os.path.join(objdir, src.replace(".cu", ".o"))
        res = subprocess.run(common + ["-c", os.path.join(CSRC, src), "-o", obj],
                             capture_output=True, text=True)
        return obj, res

    with ThreadPoolExecutor(max_workers=len(SOURCES)) as pool:
        results = list(pool.map(compile_one, SOURCES))
    for _, res in results:
        if verbose or res.returncode != 0:
            sys.stderr.write(res.stdout + res.stderr)
    if any(res.returncode != 0 for _, res in results):
        raise RuntimeError("nvcc failed compiling libginn_b200.so")
    link = subprocess.run([nvcc_path(), "-shared", "-o", LIB] + [o for o, _ in results],
                          capture_output=True, text=True)
    if link.returncode != 0:
        sys.stderr.write(link.stdout + link.stderr)
        raise RuntimeError("nvcc failed linking libginn_b200.so")
    return LIB


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(LIB)
