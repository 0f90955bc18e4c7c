"""Builds the session library in-tree with nvcc for sm_100a.

`python -m altius_b200.build` produces `altius_b200/lib/libaltius_session_cuda.so`
(the C ABI of `include/altius_session_cuda.h`). nvcc cross-compiles without a
GPU. Kernels are compiled with --fmad=false: every fused multiply-add in the
kernels is an explicit fmaf, so no rounding is added or removed relative to the
reference formulas.
"""
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIBDIR = os.path.join(HERE, "lib")
OBJDIR = os.path.join(HERE, "build")
LIB = os.path.join(LIBDIR, "libaltius_session_cuda.so")

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = (["-DAC_TC_BK=" + os.environ["AC_TC_BK"]] if "AC_TC_BK" in os.environ else []) + ["-O3", "-std=c++17", "-lineinfo", "--fmad=false", "-Xcompiler", "-fPIC,-fvisibility=hidden",
          "-Xcudafe", "--diag_suppress=177"]

SOURCES = ["session.cu", "shapes.cpp", "lower.cpp", "eltwise.cu", "rowops.cu", "movement.cu",
           "gemm_simt.cu", "gemm_tc.cu", "attention.cu", "attention_tc.cu", "noalloc.cu"]


def _newer(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(LIBDIR, exist_ok=True)
    os.makedirs(OBJDIR, exist_ok=True)
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh"))]
    headers.append(os.path.join(HERE, "..", "include", "altius_session_cuda.h"))
    objs, jobs = [], []
    for src in SOURCES:
        path = os.path.join(CSRC, src)
        obj = os.path.join(OBJDIR, src.rsplit(".", 1)[0] + ".o")
        objs.append(obj)
        if force or _newer(obj, [path] + headers):
            cmd = [NVCC, *ARCH, *COMMON, "-x", "cu", "-c", path, "-o", obj]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
            jobs.append(cmd)

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0 or verbose:
            sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
        if r.returncode != 0:
            raise RuntimeError("nvcc failed for " + cmd[-3])

    with ThreadPoolExecutor(max_workers=8) as ex:
        list(ex.map(run, jobs))
    if jobs or not os.path.exists(LIB):
        run([NVCC, *ARCH, "-shared", "-o", LIB, *objs, "-Xcompiler", "-fPIC"])
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
