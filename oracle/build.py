"""Builds the CPU oracle (test infrastructure) as oracle/libyx_oracle.so.

The flags matter for parity with the reference's Rust arithmetic: no fused multiply-add
(-ffp-contract=off), no fast-math.  -march=x86-64-v3 rather than native: the library is
built on one machine and may be loaded on another.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "yx_ref.cpp")
OUT = os.path.join(HERE, "libyx_oracle.so")
FLAGS = ["-O2", "-march=x86-64-v3", "-ffp-contract=off", "-fopenmp", "-shared", "-fPIC", "-std=c++17", "-Wall"]


def build(force: bool = False) -> str:
    deps = [SRC, os.path.join(HERE, "yx_ref.h")]
    if not force and os.path.exists(OUT) and all(os.path.getmtime(OUT) >= os.path.getmtime(d) for d in deps):
        return OUT
    cmd = ["g++", *FLAGS, "-o", OUT, SRC]
    subprocess.run(cmd, check=True)
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
