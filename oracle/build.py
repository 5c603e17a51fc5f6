"""Build recipe for the CPU oracle (test infrastructure, never shipped).

    python oracle/build.py

compiles oracle/oracle.cpp (the scalar restatement, no FMA contraction) and
oracle/cpu_kernels.cpp (the timed SIMD restatement of the reference's fastest
CPU arms, if present) into shared libraries beside the sources. The reference's
CPU path is Zig and cannot be compiled with the toolchains in this image. Its one
C++ file on this path, the CUDA kernels of its GPU provider
(src/backend/cuda/kernels.cu), does compile with nvcc:

    python oracle/build.py --ref-cuda <reference checkout>

compiles it from where it lies, together with the launch shim
oracle/ref_cuda_harness.cu, for sm_100a into oracle/_ref/libref_cuda.so (kept out
of history). Without the argument the checkout is taken from the environment
variable FUCINA_REFERENCE_DIR, else from a directory named "reference" beside the
repository; when none exists nothing is built and the users of that library
report it as unavailable.
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


def reference_dir(explicit: str | None = None) -> str | None:
    """The reference checkout that holds src/backend/cuda/kernels.cu, or None."""
    cands = [explicit, os.environ.get("FUCINA_REFERENCE_DIR"), os.path.join(os.path.dirname(HERE), os.pardir, "reference")]
    for c in cands:
        if c and os.path.exists(os.path.join(c, "src", "backend", "cuda", "kernels.cu")):
            return os.path.abspath(c)
    return None


REF_CUDA_LIB = os.path.join(HERE, "_ref", "libref_cuda.so")


def build_ref_cuda(explicit: str | None = None, force: bool = False) -> bool:
    """Compile the reference's CUDA kernels (read in place) plus the launch shim; True when the library exists."""
    ref = reference_dir(explicit)
    if ref is None:
        return os.path.exists(REF_CUDA_LIB)
    src = os.path.join(ref, "src", "backend", "cuda", "kernels.cu")
    shim = os.path.join(HERE, "ref_cuda_harness.cu")
    if not force and not _stale(REF_CUDA_LIB, [src, shim, os.path.abspath(__file__)]):
        return True
    os.makedirs(os.path.dirname(REF_CUDA_LIB), exist_ok=True)
    cmd = ["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-shared", "-Xcompiler", "-fPIC",
           "-include", src, shim, "-o", REF_CUDA_LIB]
    subprocess.check_call(cmd)
    return True


if __name__ == "__main__":
    build(force="--force" in sys.argv)
    if "--ref-cuda" in sys.argv:
        i = sys.argv.index("--ref-cuda")
        arg = sys.argv[i + 1] if i + 1 < len(sys.argv) and not sys.argv[i + 1].startswith("--") else None
        print("reference CUDA kernels:", "built" if build_ref_cuda(arg, force=True) else "no reference checkout found")
