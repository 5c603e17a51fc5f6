"""Build recipe for the CPU oracle (test infrastructure, never shipped).

    python oracle/build.py

compiles oracle/oracle.cpp (the scalar restatement, no FMA contraction) and
oracle/cpu_kernels.cpp (the timed SIMD restatement of the reference's fastest
CPU arms, if present) into shared libraries beside the sources. The reference
itself is Zig and cannot be compiled with the toolchains in this image, so no
oracle/_ref is produced.
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))


def _stale(out: str, srcs: list[str]) -> bool:
    if not os.path.exists(out):
        return True
    t = os.path.getmtime(out)
    return any(os.path.getmtime(s) > t for s in srcs)


def build(force: bool = False) -> None:
    jobs = [
        # scalar oracle: value-exact, so -O2 and no contraction
        ("liboracle.so", ["oracle.cpp"], ["-O2", "-ffp-contract=off"]),
        # timed baseline: runtime-dispatched SIMD arms; integer dots are exact
        # and the f32 epilogue keeps the oracle's association, so no contraction
        ("libcpu_kernels.so", ["cpu_kernels.cpp"], ["-O3", "-ffp-contract=off"]),
    ]
    for out, srcs, flags in jobs:
        srcs = [os.path.join(HERE, s) for s in srcs]
        if not all(os.path.exists(s) for s in srcs):
            continue
        out = os.path.join(HERE, out)
        if not force and not _stale(out, srcs + [os.path.abspath(__file__)]):
            continue
        cmd = ["g++", "-std=c++17", "-shared", "-fPIC", "-fopenmp", "-Wall", *flags, *srcs, "-o", out]
        subprocess.check_call(cmd)


if __name__ == "__main__":
    build(force="--force" in sys.argv)
