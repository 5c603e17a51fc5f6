"""fucina_b200: B200 (sm_100a) quantized-matmul provider behind fucina's GPU-offload seam.

The product is the C-ABI library `fucina_b200/lib/libfucina_b200.so`
(`include/fucina_b200.h`). This package is its Python binding: `_lib` loads the
library through ctypes, `provider` mirrors the reference provider's functions
(`src/backend/cuda.zig` pub surface) with numpy / device-pointer arguments, and
`formats` holds host-side block geometry and PTQTP plane packing.
There is no CPU fallback: importing `provider` fails loudly when the library is
missing, and every call reports declines and device errors as exceptions.
"""
from . import formats  # noqa: F401

__all__ = ["formats"]
