"""Builds libztvm_b200.so (CUDA, sm_100a only) in-tree with nvcc.

    python zero-tvm_b200/build.py [--force] [--verbose]

nvcc cross-compiles without a GPU. The library links the CUDA runtime statically and has no
Python or torch dependency; it lands in zero-tvm_b200/lib/.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB_DIR = os.path.join(HERE, "lib")
LIB = os.path.join(LIB_DIR, "libztvm_b200.so")
SOURCES = ["ztvm_api.cu", "ztvm_gemv.cu", "ztvm_gemv_mma.cu", "ztvm_gemv_tc.cu", "ztvm_gemv_tc3.cu", "ztvm_gemm.cu", "ztvm_gemm_ta.cu", "ztvm_moe_gemm.cu", "ztvm_moe_ta.cu", "ztvm_moe_ep.cu", "ztvm_moe_tc.cu", "ztvm_glue.cu"]
HEADERS = ["ztvm_device.cuh", "ztvm_tc.cuh", "ztvm_stream_mma.cuh", "ztvm_moe_plan.cuh", "ztvm_kernels.h", os.path.join("..", "..", "include", "ztvm_b200.h")]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
    "-Xcompiler", "-fPIC,-fvisibility=hidden", "--use_fast_math=false",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found: libztvm_b200.so cannot be built (there is no CPU build of this library)")


def _stale() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, s) for s in SOURCES + HEADERS] + [os.path.abspath(__file__)]
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not _stale():
        return LIB
    os.makedirs(LIB_DIR, exist_ok=True)
    flags = [f for f in NVCC_FLAGS if f != "--use_fast_math=false"] + os.environ.get("ZTVM_NVCC_EXTRA", "").split()
    objs = []
    procs = []
    for s in SOURCES:
        obj = os.path.join(LIB_DIR, s.replace(".cu", ".o"))
        cmd = [_nvcc(), *flags, "-c", os.path.join(CSRC, s), "-o", obj]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
            print(" ".join(cmd))
        procs.append((cmd, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objs.append(obj)
    for cmd, pr in procs:
        out, _ = pr.communicate()
        if verbose or pr.returncode:
            sys.stderr.write(out)
        if pr.returncode:
            raise RuntimeError("nvcc failed: " + " ".join(cmd))
    link = [_nvcc(), "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", LIB, *objs]
    subprocess.check_call(link)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
