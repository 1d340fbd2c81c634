#!/usr/bin/env python3
"""Compile the CUDA library in-tree: suzuku-engine-q4_b200/libq4cuda.so.

nvcc cross-compiles for sm_100a without a GPU.  The library is one translation
unit (csrc/q4cuda.cu includes the kernel files)."""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libq4cuda.so")

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "--compiler-options", "-fPIC", "-shared", "-Xptxas", "-v"]


def sources():
    out = []
    for root, _, files in os.walk(CSRC):
        for f in files:
            if f.endswith((".cu", ".cuh", ".h")) and f not in ("q4b_ep.cu", "tile_dot_bench.cu"):
                out.append(os.path.join(root, f))
    out.append(os.path.join(os.path.dirname(HERE), "include", "q4cuda.h"))
    return out


def build(force=False, verbose=False):
    src = sources()
    if not force and os.path.exists(LIB):
        t = os.path.getmtime(LIB)
        if all(os.path.getmtime(s) <= t for s in src):
            return LIB
    cmd = ["nvcc"] + NVCC_FLAGS + ["-o", LIB, os.path.join(CSRC, "q4cuda.cu")]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
        raise RuntimeError("nvcc failed")
    if verbose:
        sys.stderr.write(r.stderr)
    return LIB


EP_LIB = os.path.join(HERE, "libq4cuda_ep.so")


def build_ep(force=False):
    """The expert-parallel library (needs NCCL headers and libnccl)."""
    build(force)
    src = os.path.join(CSRC, "q4b_ep.cu")
    deps = [src, LIB, os.path.join(os.path.dirname(HERE), "include", "q4cuda_ep.h")]
    if not force and os.path.exists(EP_LIB) and all(os.path.getmtime(d) <= os.path.getmtime(EP_LIB) for d in deps):
        return EP_LIB
    cmd = ["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
           "--compiler-options", "-fPIC", "-shared", "-o", EP_LIB, src, "-L" + HERE, "-lq4cuda", "-lnccl",
           "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
        raise RuntimeError("nvcc failed (expert-parallel library)")
    return EP_LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
    print(build_ep(force="--force" in sys.argv))
