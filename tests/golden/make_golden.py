"""Regenerate tests/golden/*.npz.

    python tests/golden/make_golden.py [/path/to/reference]

Two fixture files are written:

* reference_goldens.npz -- the known-answer data the reference's own tests
  hold for this path, read as text from its test files (only data tables are
  extracted, no code):
    src/backend/quant/encode_golden_test.zig  input_bits (8x256 f32 bit
        patterns), q4_k_golden (8x144 B), q5_k_golden (8x176 B), q6_k_golden
        (8x210 B): ggml quantize_row_q4_K_ref / q5_K_ref / q6_K_ref outputs
    src/backend/quant/cold_tests.zig  tq2_0_dequant_golden: TQ2_0 block bytes
        with ggml's dequantised f32 bit patterns
* oracle_cases.npz -- small seeded cases run through the pinned oracle, used
  by the GPU parity tests as committed expectations (and by a CPU test that
  checks the oracle still reproduces them).
"""
from __future__ import annotations

import os
import re
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)


def _table(src: str, name: str, width_hex: int) -> np.ndarray:
    i = src.index(name)
    j = src.index("};", i)
    pat = r"0x([0-9a-fA-F]{%d})\b" % width_hex
    return np.array([int(x, 16) for x in re.findall(pat, src[i:j])], dtype=np.uint64)


def reference_goldens(ref: str) -> dict:
    enc = open(os.path.join(ref, "src/backend/quant/encode_golden_test.zig")).read()
    bits = _table(enc, "pub const input_bits", 8).astype(np.uint32).reshape(8, 256)
    q4 = _table(enc, "pub const q4_k_golden", 2).astype(np.uint8).reshape(8, 144)
    q5 = _table(enc, "pub const q5_k_golden", 2).astype(np.uint8).reshape(8, 176)
    q6 = _table(enc, "pub const q6_k_golden", 2).astype(np.uint8).reshape(8, 210)
    cold = open(os.path.join(ref, "src/backend/quant/cold_tests.zig")).read()
    i = cold.index("const tq2_0_dequant_golden")
    j = cold.index("};", i)
    body = cold[i:j]
    b0 = body.index(".bytes")
    e0 = body.index(".expected_bits")
    tq_bytes = np.array([int(x, 16) for x in re.findall(r"0x([0-9a-fA-F]{2})\b", body[b0:e0])], dtype=np.uint8)
    tq_bits = np.array([int(x, 16) for x in re.findall(r"0x([0-9a-fA-F]{8})\b", body[e0:])], dtype=np.uint32)
    assert tq_bytes.size % 66 == 0 and tq_bits.size == tq_bytes.size // 66 * 256
    return {
        "input_bits": bits,
        "q4_k_golden": q4,
        "q5_k_golden": q5,
        "q6_k_golden": q6,
        "tq2_0_bytes": tq_bytes.reshape(-1, 66),
        "tq2_0_expected_bits": tq_bits.reshape(-1, 256),
    }


def oracle_cases() -> dict:
    import oracle

    out = {}
    rng = np.random.default_rng(20251)
    # the reference's GPU parity shapes (backend/cuda.zig:3084-3088), k in blocks of 256
    for name, fmt in (("q8_0", oracle.Q8_0), ("q4_k", oracle.Q4_K), ("q5_k", oracle.Q5_K), ("q6_k", oracle.Q6_K)):
        n, k, m = 36, 512, 4
        w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
        a = rng.standard_normal((m, k)).astype(np.float32)
        blocks = oracle.quantize_rows(fmt, w)
        out[f"{name}_a"] = a
        out[f"{name}_blocks"] = blocks
        out[f"{name}_dequant"] = oracle.dequantize_rows(fmt, blocks, k)
        out[f"{name}_matmul"] = oracle.matmul(fmt, blocks, a)
    n, k, m = 36, 512, 4
    trits = rng.integers(-1, 2, size=(n, k)).astype(np.int8)
    scales = np.abs(rng.standard_normal((n, k // 256)) * 0.02).astype(np.float32)
    a = rng.standard_normal((m, k)).astype(np.float32)
    plane = oracle.pack_ptqtp_plane(trits, scales)
    out["tq2_0_trits"] = trits
    out["tq2_0_scales"] = scales
    out["tq2_0_a"] = a
    out["tq2_0_blocks"] = plane
    out["tq2_0_dequant"] = oracle.dequantize_rows(oracle.TQ2_0, plane, k)
    out["tq2_0_matmul"] = oracle.matmul(oracle.TQ2_0, plane, a)
    return out


def main() -> None:
    ref = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("FUCINA_REFERENCE", "")
    if not ref or not os.path.isdir(ref):
        sys.exit("usage: make_golden.py /path/to/the/reference checkout (or FUCINA_REFERENCE=...)")
    np.savez_compressed(os.path.join(HERE, "reference_goldens.npz"), **reference_goldens(ref))
    np.savez_compressed(os.path.join(HERE, "oracle_cases.npz"), **oracle_cases())
    print("wrote", os.listdir(HERE))


if __name__ == "__main__":
    main()
