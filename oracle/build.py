"""Build recipe for the CPU oracle (test infrastructure, never shipped code).

`build_oracle()` compiles `oracle.cpp` into `liboracle.so` beside it with the
flags the restatement depends on: no contraction of separate multiplies and
adds, no fast-math, OpenMP for the reference's thread fan-out.

The reference itself (Rust nightly with portable_simd, BLIS, clang) cannot be
compiled with the C/C++ toolchain of this image, so there is no `oracle/_ref`
binary: the restatement is the only CPU implementation available.
"""
import os
import subprocess

_HERE = os.path.dirname(os.path.abspath(__file__))
FLAGS = ["-O3", "-march=x86-64-v3", "-fopenmp", "-ffp-contract=off", "-fno-fast-math", "-fPIC",
         "-shared", "-std=c++17", "-Wall"]


def build_oracle(force: bool = False) -> str:
    src = os.path.join(_HERE, "oracle.cpp")
    out = os.path.join(_HERE, "liboracle.so")
    if not force and os.path.exists(out) and os.path.getmtime(out) >= os.path.getmtime(src):
        return out
    subprocess.check_call(["g++", *FLAGS, "-o", out, src])
    return out


if __name__ == "__main__":
    print(build_oracle(force=True))
