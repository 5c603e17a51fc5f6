"""Shared helpers for the parity tests."""
from __future__ import annotations

import numpy as np

# north_star tolerances: max relative error 1e-3 for the f32-accumulate integer
# path against the CPU-kernel oracle, 1e-2 for the bf16 tensor-core path
# against the dequantised f64 oracle.
TOL_INT8 = 1e-3
TOL_TENSOR = 1e-2


def rel_err(got: np.ndarray, want: np.ndarray) -> float:
    """max over elements of |got-want| / max(|want|, |got|, floor).

    The floor (1% of the RMS of `want`) keeps elements that cancel to ~0 from
    turning f32 summation-order noise into a meaningless ratio; the reference's
    own GPU tests use the same shape of bound with an absolute floor
    (src/backend/cuda.zig:3034).
    """
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    assert got.shape == want.shape, (got.shape, want.shape)
    assert np.isfinite(got).all(), "non-finite output"
    floor = 1e-2 * float(np.sqrt(np.mean(want**2))) + 1e-30
    den = np.maximum(np.maximum(np.abs(want), np.abs(got)), floor)
    return float(np.max(np.abs(got - want) / den))


def assert_close(got, want, tol, what=""):
    e = rel_err(got, want)
    assert e <= tol, f"{what}: max relative error {e:.3e} > {tol:g}"
    return e


def rms_err(got, want) -> tuple[float, float]:
    """(RMS of the difference, largest absolute difference), both divided by the RMS of `want`: the measure for two
    paths that round their operands differently (int8 or bf16 activations against f32 / f16 ones), where the
    difference is rounding noise proportional to the output's scale and not to each element's own size."""
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    assert got.shape == want.shape, (got.shape, want.shape)
    assert np.isfinite(got).all(), "non-finite output"
    rms = float(np.sqrt(np.mean(want**2))) + 1e-300
    d = got - want
    return float(np.sqrt(np.mean(d**2))) / rms, float(np.max(np.abs(d))) / rms


def bits_equal(a: np.ndarray, b: np.ndarray) -> bool:
    return a.shape == b.shape and np.array_equal(np.ascontiguousarray(a).view(np.uint32), np.ascontiguousarray(b).view(np.uint32))


def make_weights(fmt_name: str, n: int, k: int, seed: int):
    """Seeded N(0, 0.02) weights through the oracle quantiser (or seeded trits for the ternary formats)."""
    import oracle

    rng = np.random.default_rng(seed)
    fmt = oracle.FORMATS[fmt_name]
    if fmt_name in ("q8_0", "q4_k", "q5_k", "q6_k"):
        w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
        return oracle.quantize_rows(fmt, w)
    trits = rng.integers(-1, 2, size=(n, k)).astype(np.int8)
    if fmt_name == "tq2_0":
        scales = np.abs(rng.standard_normal((n, k // 256)) * 0.02).astype(np.float32)
        return oracle.pack_ptqtp_plane(trits, scales)
    if fmt_name == "q2_0":
        scales = np.abs(rng.standard_normal((n, k // 128)) * 0.02).astype(np.float32)
        return oracle.pack_q2_0(trits, scales)
    if fmt_name == "tq2_0_folded":
        fine = np.abs(rng.standard_normal((n, k // 256)) * 0.02).astype(np.float32)
        t2 = rng.integers(-1, 2, size=(n, k)).astype(np.int8)
        return oracle.fold_planes(oracle.pack_ptqtp_plane(trits, fine * 3), oracle.pack_ptqtp_plane(t2, fine), k)
    raise ValueError(fmt_name)


def round_bf16(a: np.ndarray) -> np.ndarray:
    """f32 -> nearest bf16 (ties to even) -> f32, the rounding the tensor-core path applies to its operands."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
    r = ((u + np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))) & np.uint32(0xFFFF0000)).astype(np.uint32)
    return r.view(np.float32)


def oracle_b(fmt: int, blocks: np.ndarray, a: np.ndarray, k: int) -> np.ndarray:
    """Oracle B at sizes the scalar C loop would take minutes for: f64 BLAS product of the oracle-dequantised
    weights and the activations, both rounded to bf16 first (the reference's GPU-test oracle,
    src/backend/cuda.zig:3016-3044, with the tensor-core operand precision)."""
    import oracle

    w = round_bf16(oracle.dequantize_rows(fmt, blocks, k)).astype(np.float64)
    return round_bf16(a).astype(np.float64) @ w.T
