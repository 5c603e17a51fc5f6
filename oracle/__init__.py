"""ctypes binding of the CPU oracle. TEST INFRASTRUCTURE ONLY.

Importable from tests/, the smoke check and the bench's CPU-baseline leg; the
shipped package never imports it.
"""
from __future__ import annotations

import ctypes
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))

Q8_0, Q6_K, Q4_K, Q5_K = 0, 1, 2, 3
TQ2_0, TQ2_0_FOLDED, Q2_0 = 16, 17, 18
FORMATS = {"q8_0": Q8_0, "q6_k": Q6_K, "q4_k": Q4_K, "q5_k": Q5_K, "tq2_0": TQ2_0, "tq2_0_folded": TQ2_0_FOLDED, "q2_0": Q2_0}
K_MULTIPLE = {Q8_0: 32, Q6_K: 256, Q4_K: 256, Q5_K: 256, TQ2_0: 256, TQ2_0_FOLDED: 256, Q2_0: 128}

_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        path = os.path.join(_HERE, "liboracle.so")
        if not os.path.exists(path):
            from . import build as _b

            _b.build()
        _lib = ctypes.CDLL(path)
        _lib.orc_row_bytes.restype = ctypes.c_size_t
        _lib.orc_row_bytes.argtypes = [ctypes.c_int, ctypes.c_size_t]
    return _lib


def _p(a: np.ndarray):
    return a.ctypes.data_as(ctypes.c_void_p)


def _sz(v):
    return ctypes.c_size_t(int(v))


def row_bytes(fmt: int, k: int) -> int:
    return int(lib().orc_row_bytes(fmt, k))


def quantize_rows(fmt: int, w: np.ndarray) -> np.ndarray:
    """[n, k] f32 -> [n, row_bytes] u8 of raw GGUF blocks."""
    w = np.ascontiguousarray(w, dtype=np.float32)
    n, k = w.shape
    assert k % K_MULTIPLE[fmt] == 0
    out = np.zeros((n, row_bytes(fmt, k)), dtype=np.uint8)
    rc = lib().orc_quantize_rows(fmt, _p(w), _sz(n), _sz(k), _p(out))
    assert rc == 0
    return out


def pack_ptqtp_plane(trits: np.ndarray, scales: np.ndarray) -> np.ndarray:
    trits = np.ascontiguousarray(trits, dtype=np.int8)
    n, k = trits.shape
    scales = np.ascontiguousarray(scales, dtype=np.float32).reshape(n, k // 256)
    out = np.zeros((n, row_bytes(TQ2_0, k)), dtype=np.uint8)
    assert lib().orc_pack_ptqtp_plane(_p(trits), _p(scales), _sz(n), _sz(k), _p(out)) == 0
    return out


def pack_q2_0(trits: np.ndarray, scales: np.ndarray) -> np.ndarray:
    trits = np.ascontiguousarray(trits, dtype=np.int8)
    n, k = trits.shape
    scales = np.ascontiguousarray(scales, dtype=np.float32).reshape(n, k // 128)
    out = np.zeros((n, row_bytes(Q2_0, k)), dtype=np.uint8)
    assert lib().orc_pack_q2_0(_p(trits), _p(scales), _sz(n), _sz(k), _p(out)) == 0
    return out


def fold_planes(p1: np.ndarray, p2: np.ndarray, k: int) -> np.ndarray:
    n = p1.shape[0]
    out = np.zeros((n, row_bytes(TQ2_0_FOLDED, k)), dtype=np.uint8)
    p1 = np.ascontiguousarray(p1)
    p2 = np.ascontiguousarray(p2)
    assert lib().orc_fold_planes(_p(p1), _p(p2), _sz(n), _sz(k), _p(out)) == 0
    return out


def dequantize_rows(fmt: int, blocks: np.ndarray, k: int) -> np.ndarray:
    blocks = np.ascontiguousarray(blocks, dtype=np.uint8)
    n = blocks.shape[0]
    assert blocks.shape[1] == row_bytes(fmt, k)
    out = np.zeros((n, k), dtype=np.float32)
    assert lib().orc_dequantize_rows(fmt, _p(blocks), _sz(n), _sz(k), _p(out)) == 0
    return out


def quantize_acts_q8_k(a: np.ndarray) -> np.ndarray:
    a = np.ascontiguousarray(a, dtype=np.float32)
    m, k = a.shape
    out = np.zeros((m, k // 256 * 292), dtype=np.uint8)
    assert lib().orc_quantize_acts_q8_k(_p(a), _sz(m), _sz(k), _p(out)) == 0
    return out


def rms_norm_mul(x: np.ndarray, w: np.ndarray, eps: float) -> np.ndarray:
    """exec/row_ops.zig:96-106 (the scalar loop): (x * scale) * w with scale = 1/sqrt(sum(x^2)/k + eps)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    w = np.ascontiguousarray(w, dtype=np.float32)
    m, k = x.shape
    out = np.zeros((m, k), dtype=np.float32)
    assert lib().orc_rms_norm_mul(_p(x), _p(w), ctypes.c_float(eps), _p(out), _sz(m), _sz(k)) == 0
    return out


def split_swiglu(gate_up: np.ndarray) -> np.ndarray:
    """exec/row_ops.zig:711-722: rows [gate: k | up: k] -> up * gate * sigmoid(gate)."""
    gate_up = np.ascontiguousarray(gate_up, dtype=np.float32)
    m, k2 = gate_up.shape
    out = np.zeros((m, k2 // 2), dtype=np.float32)
    assert lib().orc_split_swiglu(_p(gate_up), _p(out), _sz(m), _sz(k2 // 2)) == 0
    return out


def quantize_acts_q8_0(a: np.ndarray) -> np.ndarray:
    a = np.ascontiguousarray(a, dtype=np.float32)
    m, k = a.shape
    out = np.zeros((m, k // 32 * 34), dtype=np.uint8)
    assert lib().orc_quantize_acts_q8_0(_p(a), _sz(m), _sz(k), _p(out)) == 0
    return out


def matmul(fmt: int, blocks: np.ndarray, a: np.ndarray) -> np.ndarray:
    """Oracle A: the CPU-kernel replica. blocks [n, row_bytes], a [m, k] -> [m, n] f32."""
    blocks = np.ascontiguousarray(blocks, dtype=np.uint8)
    a = np.ascontiguousarray(a, dtype=np.float32)
    m, k = a.shape
    n = blocks.shape[0]
    assert blocks.shape[1] == row_bytes(fmt, k)
    c = np.zeros((m, n), dtype=np.float32)
    rc = lib().orc_matmul(fmt, _p(blocks), _sz(blocks.shape[1]), _p(a), _p(c), _sz(m), _sz(n), _sz(k))
    assert rc == 0
    return c


_fast = None


def fast_lib():
    """The SIMD restatement used as the TIMED CPU baseline (oracle/cpu_kernels.cpp), or None if it is not built."""
    global _fast
    if _fast is None:
        path = os.path.join(_HERE, "libcpu_kernels.so")
        if not os.path.exists(path):
            from . import build as _b

            _b.build()
        _fast = ctypes.CDLL(path) if os.path.exists(path) else False
    return _fast or None


def has_simd(fmt: int) -> bool:
    f = fast_lib()
    return bool(f and f.cpuk_has_simd(fmt))


def matmul_fast(fmt: int, blocks: np.ndarray, a: np.ndarray) -> np.ndarray:
    """Same values as `matmul`, computed by the runtime-dispatched SIMD arm where one exists."""
    f = fast_lib()
    if f is None:
        return matmul(fmt, blocks, a)
    blocks = np.ascontiguousarray(blocks, dtype=np.uint8)
    a = np.ascontiguousarray(a, dtype=np.float32)
    m, k = a.shape
    n = blocks.shape[0]
    assert blocks.shape[1] == row_bytes(fmt, k)
    c = np.zeros((m, n), dtype=np.float32)
    rc = f.cpuk_matmul(fmt, _p(blocks), _sz(blocks.shape[1]), _p(a), _p(c), _sz(m), _sz(n), _sz(k))
    assert rc == 0
    return c


class PackedRows:
    """The reference's load-time repack of a Q4_K / Q5_K matrix (eight rows interleaved per block, BlockQ4_Kx8 /
    BlockQ5_Kx8, src/backend/quant/types.zig:99-119) and its kernels, restated in oracle/cpu_kernels.cpp: the fastest
    CPU arm for K-quants. `PackedRows.pack` returns None where the pack does not exist (other formats, a row count that
    is not a multiple of eight, no AVX2 / F16C); results are bit-equal to `matmul`."""

    def __init__(self, handle, fmt, n, k):
        self._h, self.fmt, self.n, self.k = handle, fmt, n, k

    @classmethod
    def pack(cls, fmt: int, blocks: np.ndarray, k: int):
        f = fast_lib()
        if f is None or not hasattr(f, "cpuk_pack_rows"):
            return None
        blocks = np.ascontiguousarray(blocks, dtype=np.uint8)
        n = blocks.shape[0]
        f.cpuk_pack_rows.restype = ctypes.c_void_p
        h = f.cpuk_pack_rows(fmt, _p(blocks), _sz(blocks.shape[1]), _sz(n), _sz(k))
        return cls(h, fmt, n, k) if h else None

    @property
    def nbytes(self) -> int:
        f = fast_lib()
        f.cpuk_packed_bytes.restype = ctypes.c_size_t
        return int(f.cpuk_packed_bytes(ctypes.c_void_p(self._h)))

    def matmul(self, a: np.ndarray) -> np.ndarray:
        a = np.ascontiguousarray(a, dtype=np.float32)
        m, k = a.shape
        assert k == self.k
        c = np.zeros((m, self.n), dtype=np.float32)
        rc = fast_lib().cpuk_matmul_packed(ctypes.c_void_p(self._h), _p(a), _p(c), _sz(m))
        assert rc == 0
        return c

    def free(self) -> None:
        if self._h:
            fast_lib().cpuk_free_packed(ctypes.c_void_p(self._h))
            self._h = None

    def __del__(self):
        try:
            self.free()
        except Exception:  # noqa: BLE001 - interpreter shutdown
            pass


def moe_ffn_packed(gate: PackedRows, up: PackedRows, down: PackedRows, x, selected, weights, n_expert: int, out_pe: int) -> np.ndarray:
    """`moe_ffn` (swiglu) over packed expert stacks: the timed CPU baseline of the expert layer on its fastest arm."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    seq, hidden = x.shape
    sel = np.ascontiguousarray(selected, dtype=np.int64).reshape(seq, -1)
    top_k = sel.shape[1]
    w = np.ascontiguousarray(weights, dtype=np.float32).reshape(seq, top_k)
    out = np.zeros((seq, hidden), dtype=np.float32)
    rc = fast_lib().cpuk_moe_ffn_packed(ctypes.c_void_p(gate._h), ctypes.c_void_p(up._h), ctypes.c_void_p(down._h), _p(x), _sz(seq), _sz(hidden),
                                    _sz(out_pe), _sz(n_expert), _sz(top_k), _p(sel), _p(w), _p(out))
    assert rc == 0
    return out


def set_threads(n: int = 0) -> int:
    """Worker threads of the timed SIMD restatement (0 = all logical CPUs); returns the count in use. Set
    explicitly because launchers such as torchrun export OMP_NUM_THREADS=1."""
    f = fast_lib()
    return int(f.cpuk_set_threads(int(n))) if f is not None else 1


def threads() -> int:
    f = fast_lib()
    return int(f.cpuk_threads()) if f is not None else 1


def moe_ffn_fast(fmt, gate, up, down, x, selected, weights, n_expert, out_pe):
    """Same values as `moe_ffn`, block dots by the SIMD arms, pairs over the worker threads (the timed CPU baseline)."""
    f = fast_lib()
    if f is None:
        return moe_ffn(fmt, gate, up, down, x, selected, weights, n_expert, out_pe)
    return _moe(f.cpuk_moe_ffn, fmt, gate, up, down, x, selected, weights, n_expert, out_pe)


def matmul_ptqtp(planes: list[np.ndarray], a: np.ndarray) -> np.ndarray:
    planes = [np.ascontiguousarray(p, dtype=np.uint8) for p in planes]
    a = np.ascontiguousarray(a, dtype=np.float32)
    m, k = a.shape
    n = planes[0].shape[0]
    arr = (ctypes.c_void_p * len(planes))(*[p.ctypes.data for p in planes])
    c = np.zeros((m, n), dtype=np.float32)
    rc = lib().orc_matmul_ptqtp(arr, len(planes), _sz(planes[0].shape[1]), _p(a), _p(c), _sz(m), _sz(n), _sz(k))
    assert rc == 0
    return c


def matmul_dequant_f64(fmt: int, blocks: np.ndarray, a: np.ndarray, round_bf16: bool = False) -> np.ndarray:
    """Oracle B: f64 dot over dequantised weights (operands optionally bf16-rounded)."""
    blocks = np.ascontiguousarray(blocks, dtype=np.uint8)
    a = np.ascontiguousarray(a, dtype=np.float32)
    m, k = a.shape
    n = blocks.shape[0]
    c = np.zeros((m, n), dtype=np.float64)
    rc = lib().orc_matmul_dequant_f64(
        fmt, _p(blocks), _sz(blocks.shape[1]), _p(a), _p(c), _sz(m), _sz(n), _sz(k), 1 if round_bf16 else 0
    )
    assert rc == 0
    return c


def block_dot(fmt: int, wblock: np.ndarray, ablock: np.ndarray) -> np.float32:
    wblock = np.ascontiguousarray(wblock, dtype=np.uint8)
    ablock = np.ascontiguousarray(ablock, dtype=np.uint8)
    f = lib().orc_block_dot
    f.restype = ctypes.c_float
    return np.float32(f(fmt, _p(wblock), _p(ablock)))


def router_topk(logits: np.ndarray, k: int, normalize: bool = True):
    logits = np.ascontiguousarray(logits, dtype=np.float32)
    rows, experts = logits.shape
    sel = np.zeros((rows, k), dtype=np.int64)
    w = np.zeros((rows, k), dtype=np.float32)
    assert lib().orc_router_topk(_p(logits), _sz(rows), _sz(experts), _sz(k), int(normalize), _p(sel), _p(w)) == 0
    return sel, w


def route_plan(selected: np.ndarray, n_expert: int):
    sel = np.ascontiguousarray(selected, dtype=np.int64).reshape(-1)
    pairs = sel.size
    count = np.zeros(n_expert, dtype=np.int64)
    offset = np.zeros(n_expert + 1, dtype=np.int64)
    order = np.zeros(pairs, dtype=np.int64)
    inv = np.zeros(pairs, dtype=np.int64)
    rc = lib().orc_route_plan(_p(sel), _sz(pairs), _sz(n_expert), _p(count), _p(offset), _p(order), _p(inv))
    assert rc == 0
    return count, offset, order, inv


GATED_SWIGLU, GATED_GEGLU, GATED_SWIGLU_CLAMP10, GATED_GLU, GATED_SITU = range(5)


def moe_ffn_bf16(fmt, gate, up, down, x, selected, weights, n_expert, out_pe, gated_op=0, fmt_down=None):
    """Oracle B of the expert layer: bf16 operands, f64 dots, f32 activation (the tensor-core arm's reference)."""
    fn = lambda *a: lib().orc_moe_ffn_bf16_gated(fmt, fmt if fmt_down is None else fmt_down, gated_op, *a[1:])  # noqa: E731
    return _moe(fn, fmt, gate, up, down, x, selected, weights, n_expert, out_pe)


def moe_ffn(fmt, gate, up, down, x, selected, weights, n_expert, out_pe, gated_op=0, fmt_down=None):
    """Oracle A of the expert layer (exec/moe.zig:890-920, :1287-1292); `gated_op` follows backend/ops.zig:89-107,
    `fmt_down` is the down tensor's format when it differs from gate/up."""
    fn = lambda *a: lib().orc_moe_ffn_gated(fmt, fmt if fmt_down is None else fmt_down, gated_op, *a[1:])  # noqa: E731
    return _moe(fn, fmt, gate, up, down, x, selected, weights, n_expert, out_pe)


def _moe(fn, fmt, gate, up, down, x, selected, weights, n_expert, out_pe):
    """gate/up: [E*out_pe, rb(hidden)] u8; down: [E*hidden, rb(out_pe)] u8; x [seq, hidden]."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    seq, hidden = x.shape
    sel = np.ascontiguousarray(selected, dtype=np.int64).reshape(seq, -1)
    top_k = sel.shape[1]
    w = np.ascontiguousarray(weights, dtype=np.float32).reshape(seq, top_k)
    gate = np.ascontiguousarray(gate)
    up = np.ascontiguousarray(up)
    down = np.ascontiguousarray(down)
    out = np.zeros((seq, hidden), dtype=np.float32)
    rc = fn(
        fmt, _p(gate), _p(up), _p(down), _p(x), _sz(seq), _sz(hidden), _sz(out_pe), _sz(n_expert), _sz(top_k),
        _p(sel), _p(w), _p(out),
    )
    assert rc == 0
    return out


def moe_ffn_ptqtp(gate_planes, up_planes, down_planes, x, selected, weights, n_expert, out_pe, gated_op=0):
    """Expert layer over multi-plane ternary experts (exec/moe.zig:51-78, :591-631): lists of K TQ2_0 plane stacks
    per projection, plane dots summed per element in plane order."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    seq, hidden = x.shape
    sel = np.ascontiguousarray(selected, dtype=np.int64).reshape(seq, -1)
    top_k = sel.shape[1]
    w = np.ascontiguousarray(weights, dtype=np.float32).reshape(seq, top_k)
    keep = [[np.ascontiguousarray(p, dtype=np.uint8) for p in planes] for planes in (gate_planes, up_planes, down_planes)]
    K = len(keep[0])
    arrs = [(ctypes.c_void_p * K)(*[p.ctypes.data for p in planes]) for planes in keep]
    out = np.zeros((seq, hidden), dtype=np.float32)
    rc = lib().orc_moe_ffn_ptqtp(K, gated_op, arrs[0], arrs[1], arrs[2], _p(x), _sz(seq), _sz(hidden), _sz(out_pe), _sz(n_expert),
                                 _sz(top_k), _p(sel), _p(w), _p(out))
    assert rc == 0
    return out
