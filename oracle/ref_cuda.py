"""ctypes binding of oracle/_ref/libref_cuda.so: the reference's own CUDA kernels
(src/backend/cuda/kernels.cu, compiled unmodified for sm_100a by oracle/build.py)
behind a launch shim. Test and bench infrastructure only: a second checker beside
the CPU oracle and the "reference kernels on this GPU" column of the bench. The
product never loads it.

Pointers are raw device addresses (torch tensors' data_ptr()); `stream` is a CUDA
stream handle (0 = the legacy default stream).
"""
from __future__ import annotations

import ctypes
import os

from .build import REF_CUDA_LIB

_lib = None

# the reference's QFormat order (backend/cuda.zig QFormat; kernels.cu kernel tables)
FORMATS = {"q8_0": 0, "q6_k": 1, "q4_k": 2, "q5_k": 3}


def available() -> bool:
    return os.path.exists(REF_CUDA_LIB)


def lib():
    global _lib
    if _lib is None:
        if not available():
            raise RuntimeError("oracle/_ref/libref_cuda.so is missing: run `python oracle/build.py --ref-cuda <reference checkout>`")
        L = ctypes.CDLL(REF_CUDA_LIB)
        vp, ull, i32 = ctypes.c_void_p, ctypes.c_ulonglong, ctypes.c_int
        L.refk_gemv.argtypes = [i32, vp, vp, vp, i32, i32, i32, ull, vp]
        L.refk_gemv.restype = i32
        L.refk_plan.argtypes = [i32, i32, ctypes.c_longlong, ctypes.c_longlong, ctypes.c_longlong, i32,
                                ctypes.POINTER(i32), ctypes.POINTER(i32)]
        L.refk_plan.restype = None
        L.refk_mul_mm.argtypes = [i32, vp, vp, vp, i32, vp, i32, i32, ull, ull, vp, i32, ull, i32, vp]
        L.refk_mul_mm.restype = i32
        L.refk_attn_fwd.argtypes = [i32, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, ctypes.c_float, i32, i32, vp]
        L.refk_attn_fwd.restype = i32
        _lib = L
    return _lib


def _check(rc: int, what: str) -> None:
    if rc != 0:
        raise RuntimeError(f"reference kernel launch refused ({what}): rc={rc}")


def gemv(fmt: int, w_ptr: int, x_ptr: int, y_ptr: int, k: int, n: int, m: int, nb01: int, stream: int = 0) -> None:
    """y[m, n] = x[m, k] . dequant(W[n, k])^T with the reference's decode kernel (m <= 8)."""
    _check(lib().refk_gemv(fmt, w_ptr, x_ptr, y_ptr, k, n, m, nb01, stream), "gemv")


def plan(fmt: int, sm_count: int, grid_x: int, n: int, k: int, allow_split_k: bool = True) -> tuple[int, int]:
    """(n_tile, split_k) the reference's host code would choose for a table of grid_x row tiles."""
    nt, sk = ctypes.c_int(0), ctypes.c_int(0)
    lib().refk_plan(fmt, sm_count, grid_x, n, k, int(allow_split_k), ctypes.byref(nt), ctypes.byref(sk))
    return nt.value, sk.value


def mul_mm(fmt: int, w_ptr: int, a_ptr: int, tiles_ptr: int, n_tiles: int, dst_ptr: int, k: int, n: int, nb01: int, nb02: int,
           partial_ptr: int = 0, split_k: int = 1, partial_stride: int = 0, n_tile: int = 64, stream: int = 0) -> None:
    """One grouped tensor-core launch over a device table of int32 {expert, base_row, m, tile_m} entries."""
    _check(lib().refk_mul_mm(fmt, w_ptr, a_ptr, tiles_ptr, n_tiles, dst_ptr, k, n, nb01, nb02, partial_ptr or None, split_k,
                             partial_stride, n_tile, stream), "mul_mm")


def attn_fwd(kv_is_f16: bool, q_ptr: int, k_ptr: int, v_ptr: int, o_ptr: int, stats_ptr: int, kvmap_ptr: int, q_seq: int, kv_seq: int,
             heads: int, kv_heads: int, d: int, source_offset: int, scale: float, window: int, causal: bool, stream: int = 0) -> None:
    """The reference's streaming attention forward (one warp per query row and head)."""
    _check(lib().refk_attn_fwd(int(kv_is_f16), q_ptr, k_ptr, v_ptr, o_ptr, stats_ptr or None, kvmap_ptr, q_seq, kv_seq, heads, kv_heads, d,
                               source_offset, scale, window, int(causal), stream), "attn_fwd")


def dense_tiles(m: int) -> list[list[int]]:
    """The tile table of one dense product of m activation rows (backend/cuda.zig:2075-2090)."""
    return [[0, 0, m, t] for t in range((m + 31) // 32)]


def grouped_tiles(counts) -> list[list[int]]:
    """Tile table of a grouped product: expert e owns counts[e] consecutive rows of the panel, 32 rows per tile
    (backend/cuda.zig:2244-2333 takes this table from the host's route plan)."""
    tiles, base = [], 0
    for e, c in enumerate(counts):
        c = int(c)
        for t in range((c + 31) // 32):
            tiles.append([e, base, c, t])
        base += c
    return tiles
