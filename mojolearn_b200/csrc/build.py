"""Compile libb200i.so (the CUDA kernels and their C ABI) for sm_100a, in tree.

    python -m mojolearn_b200.csrc.build [--force] [--verbose]

nvcc cross-compiles without a GPU. The flags are part of the numerical
contract: no multiply-add contraction by the compiler (-fmad=false), IEEE
subnormals (-ftz=false), IEEE division and square root, no fast-math. Every
fused multiply-add in the kernels is an explicit fma.rn.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(HERE, "libb200i.so")
#: the negative-control build: every window admitted (-DB200I_SABOTAGE_ADMIT_ALWAYS); loaded only by the tests
SABOTAGE_LIB = os.path.join(HERE, "libb200i_sabotage_admit.so")
SOURCES = ["b200i.cu"]
HEADERS = sorted(f for f in os.listdir(HERE) if f.endswith(".cuh")) + [os.path.join("..", "..", "include", "b200i.h")]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-fmad=false", "-ftz=false", "-prec-div=true", "-prec-sqrt=true",
    "-shared", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=default", "-cudart", "shared",
]


def stale(lib=LIB):
    if not os.path.exists(lib):
        return True
    t = os.path.getmtime(lib)
    deps = [os.path.join(HERE, s) for s in SOURCES + HEADERS] + [os.path.abspath(__file__)]
    return any(os.path.exists(d) and os.path.getmtime(d) > t for d in deps)


def build(force=False, verbose=False, sabotage=False):
    lib = SABOTAGE_LIB if sabotage else LIB
    if not force and not stale(lib):
        return lib
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    cmd = [nvcc] + NVCC_FLAGS + (["-DB200I_SABOTAGE_ADMIT_ALWAYS"] if sabotage else []) + (["-Xptxas", "-v"] if verbose else []) \
        + [os.path.join(HERE, s) for s in SOURCES] + ["-o", lib]
    subprocess.run(cmd, check=True)
    return lib


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv, sabotage="--sabotage" in sys.argv))
