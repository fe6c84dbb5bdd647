"""Compiles the oracle's C restatement (w8a8_oracle.c -> libw8a8_oracle.so).

TEST INFRASTRUCTURE, not part of the product.  Usage: python oracle/build.py [--force]
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "w8a8_oracle.c")
OUT = os.path.join(HERE, "libw8a8_oracle.so")
CFLAGS = ["-O3", "-mavx2", "-mfma", "-fopenmp", "-ffp-contract=off", "-fPIC",
          "-fvisibility=hidden", "-std=gnu11"]


def build(force=False):
    if (not force and os.path.exists(OUT)
            and os.path.getmtime(OUT) >= max(os.path.getmtime(SRC), os.path.getmtime(__file__))):
        return OUT
    # The system gcc: an alternative toolchain on PATH may lack libgomp.
    cc = "/usr/bin/gcc" if os.path.exists("/usr/bin/gcc") else "gcc"
    subprocess.check_call([cc] + CFLAGS + ["-shared", "-o", OUT, SRC, "-lm"])
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
