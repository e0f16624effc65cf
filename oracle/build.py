"""Build the CPU oracle library (test infrastructure, never the product path).

`python oracle/build.py` compiles oracle.c (the scalar restatement of the
reference's normative host algorithm) and cpu_rows.c (its AVX2 CPU-speed form)
into oracle/liboracle.so. The flags are part of the arithmetic: no contraction
by the compiler, no fast-math; the one fused multiply-add is fmaf().
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(HERE, "liboracle.so")
SOURCES = ["oracle.c", "cpu_rows.c", "decoder_oracle.c"]
FLAGS = ["-O2", "-std=gnu11", "-fPIC", "-shared", "-ffp-contract=off", "-fno-fast-math", "-fno-unsafe-math-optimizations",
         "-frounding-math", "-mfma", "-mavx2", "-fvisibility=hidden", "-Wall", "-Wno-unused-function"]


def build(force=False):
    srcs = [os.path.join(HERE, s) for s in SOURCES if os.path.exists(os.path.join(HERE, s))]
    if not force and os.path.exists(LIB) and all(os.path.getmtime(LIB) >= os.path.getmtime(s) for s in srcs):
        return LIB
    cmd = ["gcc"] + FLAGS + srcs + ["-o", LIB, "-lm", "-lpthread"]
    subprocess.run(cmd, check=True)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
