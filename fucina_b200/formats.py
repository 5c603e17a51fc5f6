"""Host-side block geometry and PTQTP plane packing (numpy, no GPU needed).

Format ids keep the reference's `QFormat` values (src/backend/cuda.zig:1486)
and add the ternary formats clear of both providers' enums.
"""
from __future__ import annotations

import numpy as np

Q8_0, Q6_K, Q4_K, Q5_K = 0, 1, 2, 3
TQ2_0, TQ2_0_FOLDED, Q2_0 = 16, 17, 18

NAMES = {Q8_0: "q8_0", Q6_K: "q6_k", Q4_K: "q4_k", Q5_K: "q5_k", TQ2_0: "tq2_0", TQ2_0_FOLDED: "tq2_0_folded", Q2_0: "q2_0"}
BY_NAME = {v: k for k, v in NAMES.items()}
# (elements per block, GGUF bytes per block): src/dtype.zig:78-86, :128-139, :215-218; quant/types.zig:177-180
BLOCK = {Q8_0: (32, 34), Q6_K: (256, 210), Q4_K: (256, 144), Q5_K: (256, 176), TQ2_0: (256, 66), TQ2_0_FOLDED: (256, 130), Q2_0: (128, 34)}


def row_bytes(fmt: int, k: int) -> int:
    elems, nbytes = BLOCK[fmt]
    if k % elems:
        raise ValueError(f"k={k} is not a whole number of {elems}-element blocks")
    return k // elems * nbytes


def pack_ptqtp_plane(trits: np.ndarray, scales: np.ndarray) -> np.ndarray:
    """One PTQTP plane as TQ2_0 blocks (src/ptqtp.zig:684-697 `packBlock`).

    trits [n, k] in {-1, 0, +1}; scales [n, k/256] f32 (stored as f16).
    Byte m of half-group hg holds elements hg*128 + n*32 + m as code = trit + 1
    in bits 2n+1:2n; the f16 scale follows the 64 payload bytes.
    """
    trits = np.asarray(trits, dtype=np.int8)
    n, k = trits.shape
    if k % 256:
        raise ValueError("k must be a multiple of 256")
    bpr = k // 256
    codes = (trits.reshape(n, bpr, 2, 4, 32) + 1).astype(np.uint8)  # [n, blk, hg, crumb, m]
    qs = codes[:, :, :, 0] | (codes[:, :, :, 1] << 2) | (codes[:, :, :, 2] << 4) | (codes[:, :, :, 3] << 6)
    out = np.empty((n, bpr, 66), dtype=np.uint8)
    out[:, :, :64] = qs.reshape(n, bpr, 64)
    d = np.asarray(scales, dtype=np.float32).reshape(n, bpr).astype(np.float16)
    out[:, :, 64:] = d.view(np.uint8).reshape(n, bpr, 2)
    return out.reshape(n, bpr * 66)


def pack_q2_0(trits: np.ndarray, scales: np.ndarray) -> np.ndarray:
    """Q2_0 g128 blocks (src/dtype.zig:78-81; decode law src/backend/quant/cold.zig:285-301)."""
    trits = np.asarray(trits, dtype=np.int8)
    n, k = trits.shape
    if k % 128:
        raise ValueError("k must be a multiple of 128")
    bpr = k // 128
    codes = (trits.reshape(n, bpr, 32, 4) + 1).astype(np.uint8)
    qs = codes[..., 0] | (codes[..., 1] << 2) | (codes[..., 2] << 4) | (codes[..., 3] << 6)
    out = np.empty((n, bpr, 34), dtype=np.uint8)
    d = np.asarray(scales, dtype=np.float32).reshape(n, bpr).astype(np.float16)
    out[:, :, :2] = d.view(np.uint8).reshape(n, bpr, 2)
    out[:, :, 2:] = qs
    return out.reshape(n, bpr * 34)


def fold_planes(coarse: np.ndarray, fine: np.ndarray, k: int) -> np.ndarray:
    """Row-major fold of two tie-fitted TQ2_0 planes (src/backend/quant/ternary.zig:707-735).

    cu = 3*code_coarse + code_fine in 0..8; byte s*16+j = cu(s*32+j) | cu(s*32+16+j) << 4;
    the folded block keeps the fine plane's f16 scale.
    """
    n = coarse.shape[0]
    bpr = k // 256

    def codes(plane):
        qs = plane.reshape(n, bpr, 66)[:, :, :64].reshape(n, bpr, 2, 32)
        c = np.stack([(qs >> (2 * j)) & 3 for j in range(4)], axis=3)  # [n, blk, hg, crumb, m]
        return c.reshape(n, bpr, 256)

    cu = (3 * codes(coarse) + codes(fine)).astype(np.uint8).reshape(n, bpr, 8, 2, 16)
    qs = cu[:, :, :, 0] | (cu[:, :, :, 1] << 4)
    out = np.empty((n, bpr, 130), dtype=np.uint8)
    out[:, :, :128] = qs.reshape(n, bpr, 128)
    out[:, :, 128:] = fine.reshape(n, bpr, 66)[:, :, 64:]
    return out.reshape(n, bpr * 130)
