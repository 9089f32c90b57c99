"""Builds libava_engine.so (the C-ABI library of include/ava_engine.h) in-tree with nvcc for sm_100a.

-fmad=false on the device side and -ffp-contract=off on the host side: a multiply-add is fused only where the source
says so, which is what makes the kernels return the bits of the reference's ordered sums.
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libava_engine.so")
SOURCES = ["engine.cu", "ops.cu", "k_gemm.cu", "k_gemm2.cu", "k_stream.cu", "k_rows.cu", "k_delta.cu", "k_engram.cu", "k_tc.cu", "k_tcb.cu", "k_chunk.cu", "k_eattn.cu", "k_sample.cu", "k_parts.cu", "k_cb.cu", "static_entry.cu", "nccl_dl.cpp", "loader.cpp", "generate.cpp", "state_io.cpp", "trace.cpp"]
HEADERS = sorted(f for f in os.listdir(CSRC) if f.endswith((".h", ".cuh"))) + [os.path.join("..", "..", "include", "ava_engine.h")]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-fmad=false",
              "-Xcompiler", "-fPIC,-ffp-contract=off,-O2", "-ccbin", "g++"]


def _stale() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, s) for s in SOURCES + HEADERS] + [os.path.abspath(__file__)]
    return any(os.path.getmtime(p) > t for p in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    if not (force or _stale()):
        return LIB
    objdir = os.path.join(HERE, "build")
    os.makedirs(objdir, exist_ok=True)
    objs = []
    procs = []
    for s in SOURCES:
        o = os.path.join(objdir, os.path.splitext(s)[0] + ".o")
        objs.append(o)
        cmd = ["nvcc"] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-c", os.path.join(CSRC, s), "-o", o]
        procs.append((s, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    for s, p in procs:
        out, _ = p.communicate()
        if verbose or p.returncode:
            sys.stderr.write(out)
        if p.returncode:
            raise RuntimeError(f"nvcc failed on {s}")
    subprocess.check_call(["nvcc", "-shared", "-o", LIB] + objs + ["-ldl", "-Wno-deprecated-gpu-targets"])
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
