"""Builds libaussm_b200.so in-tree with nvcc for sm_100a.

Usage:  python -m aussm_b200.build [--verbose]
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libaussm_b200.so")
SOURCES = ["scan_unitary.cu", "projection.cu", "gemm_split3.cu", "scan_s6.cu", "scan_s6_wide.cu", "scan_complex.cu", "api.cu", "api_s6.cu", "api_complex.cu", "noalloc.cu", "block_stages.cu"]
HEADERS = ["common.cuh", "scan_unitary.cuh", "projection.cuh", "gemm_split3.cuh", "host_common.cuh", "scan_s6.cuh", "scan_complex.cuh", os.path.join("..", "..", "include", "aussm_b200.h")]


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found (set NVCC)")
    return cand


def _stale() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, s) for s in SOURCES + HEADERS] + [os.path.abspath(__file__)]
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile every CUDA source into one shared library; returns its path."""
    if not force and not _stale():
        return LIB
    objdir = os.path.join(HERE, "build")
    os.makedirs(objdir, exist_ok=True)
    common = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC,-O3,-Wall", "-I", os.path.join(HERE, "..", "include")]
    if verbose:
        common += ["-Xptxas", "-v"]
    procs = []
    objs = []
    for s in SOURCES:
        o = os.path.join(objdir, s.replace(".cu", ".o"))
        objs.append(o)
        cmd = [_nvcc(), *common, "-c", os.path.join(CSRC, s), "-o", o]
        procs.append((cmd, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    for cmd, p in procs:
        out, _ = p.communicate()
        if verbose or p.returncode:
            print(out)
        if p.returncode:
            raise RuntimeError("nvcc failed: " + " ".join(cmd))
    cuda_lib = os.path.join(os.path.dirname(os.path.dirname(_nvcc())), "lib64")
    link = [_nvcc(), "-shared", "-o", LIB, *objs, "-L", cuda_lib, "-lcudart",
            "-Xlinker", "-rpath=" + cuda_lib]
    r = subprocess.run(link, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode:
        print(r.stdout)
        raise RuntimeError("link failed: " + " ".join(link))
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
