"""Builds the native libraries in-tree.

  libhemmer_b200.so  CUDA kernels + the C ABI of include/hemmer_b200.h   (nvcc, sm_100a)
  libhellm_b200.so   C++ HELLM::HEMMer layer over that C ABI             (g++)

Run as a script (``python build.py``) or call :func:`build`.
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
ROOT = os.path.dirname(HERE)
NVCC = os.environ.get("HB_NVCC", "/usr/local/cuda/bin/nvcc")
GXX = "/usr/bin/g++"

CUDA_LIB = os.path.join(HERE, "libhemmer_b200.so")
HELLM_LIB = os.path.join(HERE, "libhellm_b200.so")


def _newer(target, sources):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def _run(cmd):
    print("+", " ".join(cmd), flush=True)
    subprocess.check_call(cmd)


def build(force: bool = False, verbose_ptxas: bool = False) -> None:
    cu_src = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cu", ".cuh", ".hpp"))]
    cu_src.append(os.path.join(ROOT, "include", "hemmer_b200.h"))
    if force or _newer(CUDA_LIB, cu_src):
        cmd = [NVCC, "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-shared", "-ccbin", GXX,
               "-Xcompiler", "-fPIC,-ffp-contract=off,-O2",
               "-o", CUDA_LIB, os.path.join(CSRC, "hemmer_b200.cu"), "-ldl"]
        if verbose_ptxas:
            cmd.insert(1, "-Xptxas=-v")
        _run(cmd)
    hellm_dir = os.path.join(CSRC, "hellm")
    if os.path.isdir(hellm_dir):
        cpp = [os.path.join(hellm_dir, f) for f in os.listdir(hellm_dir)]
        srcs = [f for f in cpp if f.endswith(".cpp")]
        if srcs and (force or _newer(HELLM_LIB, cpp + [CUDA_LIB])):
            _run([GXX, "-O2", "-std=c++17", "-fPIC", "-shared", "-ffp-contract=off", "-Wall", "-I", os.path.join(ROOT, "include"), "-I", hellm_dir,
                  "-o", HELLM_LIB, *srcs, "-L", HERE, "-lhemmer_b200", "-Wl,-rpath,$ORIGIN"])


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose_ptxas="-v" in sys.argv)
