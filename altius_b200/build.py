"""Builds the session library in-tree with nvcc for sm_100a.

`python -m altius_b200.build` produces `altius_b200/lib/libaltius_session_cuda.so`
(the C ABI of `include/altius_session_cuda.h`). nvcc cross-compiles without a
GPU. Kernels are compiled with --fmad=false: every fused multiply-add in the
kernels is an explicit fmaf, so no rounding is added or removed relative to the
reference formulas.
"""
import hashlib
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
           "gemm_simt.cu", "gemm_tc.cu", "attention.cu", "attention_tc.cu", "attention_tc16.cu", "noalloc.cu",
           "model.cpp", "onnx_load.cpp", "passes.cpp"]


def _fingerprint(cmd, deps):
    """Hash of the compile command and of the contents of everything it reads: an object is
    rebuilt whenever its source, any header or a flag differs from what it was built from
    (modification times are not trusted; prebuilt objects travel between machines)."""
    h = hashlib.sha256(" ".join(cmd).encode())
    for d in sorted(deps):
        with open(d, "rb") as f:
            h.update(hashlib.sha256(f.read()).digest())
    return h.hexdigest()


def _stale(obj, stamp, fingerprint):
    if not os.path.exists(obj) or not os.path.exists(stamp):
        return True
    with open(stamp) as f:
        return f.read().strip() != fingerprint


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(LIBDIR, exist_ok=True)
    os.makedirs(OBJDIR, exist_ok=True)
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh"))]
    headers.append(os.path.join(HERE, "..", "include", "altius_session_cuda.h"))
    objs, jobs = [], []
    for src in SOURCES:
        path = os.path.join(CSRC, src)
        obj = os.path.join(OBJDIR, src.rsplit(".", 1)[0] + ".o")
        stamp = obj + ".stamp"
        objs.append(obj)
        cmd = [NVCC, *ARCH, *COMMON, "-x", "cu", "-c", path, "-o", obj]
        fp = _fingerprint(cmd, [path] + headers)
        if force or verbose or _stale(obj, stamp, fp):
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
            jobs.append((cmd, stamp, fp))

    def run(job):
        cmd, stamp, fp = job
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0 or verbose:
            sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
        if r.returncode != 0:
            raise RuntimeError("nvcc failed for " + cmd[-3])
        if stamp:
            with open(stamp, "w") as f:
                f.write(fp)

    with ThreadPoolExecutor(max_workers=8) as ex:
        list(ex.map(run, jobs))
    # The library records what it was linked from in the same way.
    link = [NVCC, *ARCH, "-shared", "-o", LIB, *objs, "-Xcompiler", "-fPIC"]
    lib_fp = hashlib.sha256(" ".join(link).encode())
    for o in objs:
        with open(o + ".stamp") as f:
            lib_fp.update(f.read().encode())
    lib_stamp = os.path.join(OBJDIR, "lib.stamp")
    if jobs or _stale(LIB, lib_stamp, lib_fp.hexdigest()):
        run((link, lib_stamp, lib_fp.hexdigest()))
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
