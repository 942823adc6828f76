"""Builds ``libsynaptik_cuda.so`` in-tree with nvcc for sm_100a (cross-compiles without a GPU)."""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB_DIR = os.path.join(HERE, os.environ.get("SYNAPTIK_LIB_DIR", "lib"))
LIB_PATH = os.path.join(LIB_DIR, "libsynaptik_cuda.so")
SOURCES = ["program.cpp", "lowering.cpp", "kernels_rowwise.cu", "kernels_gemm.cu", "kernels_skinny.cu", "runtime.cu"]
HEADERS = ["program.hpp", "lowering.hpp", "kernels.hpp", os.path.join("..", "..", "include", "synaptik_cuda.h")]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC,-fvisibility=hidden,-Wall", "--expt-relaxed-constexpr"]


def _nvcc() -> str:
    for candidate in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if candidate and (os.path.isabs(candidate) and os.path.exists(candidate) or not os.path.isabs(candidate)):
            return candidate
    raise RuntimeError("nvcc not found")


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(LIB_DIR, exist_ok=True)
    extra = os.environ.get("SYNAPTIK_NVCC_EXTRA", "").split()
    inputs = [os.path.join(CSRC, s) for s in SOURCES + HEADERS]
    newest = max(os.path.getmtime(p) for p in inputs)
    objects = []
    procs = []
    for source in SOURCES:
        obj = os.path.join(LIB_DIR, os.path.splitext(source)[0] + ".o")
        objects.append(obj)
        if force or not os.path.exists(obj) or os.path.getmtime(obj) < newest:
            cmd = [_nvcc(), *NVCC_FLAGS, *extra, "-x", "cu", "-c", os.path.join(CSRC, source), "-o", obj]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
            procs.append((source, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = False
    for source, proc in procs:
        out, _ = proc.communicate()
        if out.strip() and (verbose or proc.returncode):
            sys.stderr.write(out)
        failed |= proc.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed")
    if procs or not os.path.exists(LIB_PATH):
        link = [_nvcc(), "-shared", "-o", LIB_PATH, *objects, "-gencode", "arch=compute_100a,code=sm_100a",
                "-cudart", "static", "-ldl", "-lpthread", "-Xlinker", "--no-undefined"]
        subprocess.run(link, check=True)
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
