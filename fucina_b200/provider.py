"""Python mirror of the provider interface (reference `src/backend/cuda.zig` pub surface).

Function names follow the reference (`gemmQuantNt`, `gemmQuantNtAsync`,
`gemmQGroupedNt`, `allocResidentBytes`, `shouldUseGpu*` ...) in snake case;
arguments keep their meaning. Where the reference returns `false`/`null`
("the GPU did not run, nothing was written") these raise `Declined`; a device
failure after submission raises `DeviceError`. Nothing here computes on the
CPU.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

from . import formats
from ._lib import QmmTile, load

MODE_AUTO, MODE_INT8, MODE_TENSOR = 0, 1, 2


class Declined(RuntimeError):
    """The provider refused before any side effect (the reference's `false`)."""

    def __init__(self, code: int, msg: str):
        super().__init__(f"declined ({code}): {msg}")
        self.code = code


class DeviceError(RuntimeError):
    """A CUDA failure after submission (a failed accelerator.Work)."""

    def __init__(self, code: int, msg: str):
        super().__init__(f"device error ({code}): {msg}")
        self.code = code


def last_error() -> str:
    buf = C.create_string_buffer(512)
    load().fq_last_error(buf, 512)
    return buf.value.decode(errors="replace")


def _check(rc: int) -> None:
    if rc == 0:
        return
    if rc > 0:
        raise Declined(rc, last_error())
    raise DeviceError(rc, last_error())


def _vp(x) -> C.c_void_p:
    """numpy array, torch tensor, int address or None -> void*."""
    if x is None:
        return C.c_void_p(0)
    if isinstance(x, np.ndarray):
        return C.c_void_p(x.ctypes.data)
    if isinstance(x, int):
        return C.c_void_p(x)
    if hasattr(x, "data_ptr"):
        return C.c_void_p(x.data_ptr())
    raise TypeError(type(x))


def init(device: int = -1) -> None:
    _check(load().fq_init(device))


def device_name() -> str:
    return load().fq_device_name().decode()


def sm_count() -> int:
    return load().fq_sm_count()


def stream_ptr() -> int:
    return int(load().fq_stream() or 0)


def synchronize() -> None:
    _check(load().fq_synchronize())


def host_register(a: np.ndarray) -> None:
    """`ensureHostRegistered` (src/backend/cuda.zig:1047-1082): page-lock a numpy array's storage for its lifetime."""
    _check(load().fq_host_register(_vp(a), a.nbytes))


def host_unregister(a: np.ndarray) -> None:
    _check(load().fq_host_unregister(_vp(a)))


def trace_counters() -> dict:
    arr = (C.c_uint64 * 8)()
    load().fq_trace_counters(arr)
    keys = ["calls", "launches", "h2d_bytes", "d2h_bytes", "resident_hits", "resident_adopts", "gate_pass", "gate_fail"]
    return dict(zip(keys, [int(v) for v in arr]))


def kernel_timing(enable: bool) -> None:
    """Bracket every decode-kernel launch with CUDA events (off by default)."""
    load().fq_trace_kernel_timing(int(enable))


def kernel_times() -> tuple[float, int]:
    """(summed device milliseconds, launches) of the decode kernel since the last query."""
    ms, n = C.c_double(), C.c_uint64()
    _check(load().fq_trace_kernel_times(C.byref(ms), C.byref(n)))
    return ms.value, int(n.value)


# --------------------------------------------------------------------------- weights
class Weights:
    """Device-resident weights in the gpu_formats layout (`fq_weights`)."""

    def __init__(self, handle: int, fmt: int, n: int, k: int, n_mats: int):
        self.handle, self.fmt, self.n, self.k, self.n_mats = handle, fmt, n, k, n_mats

    @classmethod
    def upload(cls, fmt: int, blocks: np.ndarray, n: int, k: int, n_mats: int = 1) -> "Weights":
        """blocks: uint8 raw GGUF rows, [n_mats*n, row_bytes] (dense strides)."""
        blocks = np.ascontiguousarray(blocks, dtype=np.uint8)
        nb01 = formats.row_bytes(fmt, k)
        assert blocks.size == n_mats * n * nb01, (blocks.size, n_mats, n, nb01)
        h = C.c_void_p()
        _check(load().fq_weights_upload(fmt, _vp(blocks), nb01, nb01 * n, n, k, n_mats, C.byref(h)))
        return cls(h.value, fmt, n, k, n_mats)

    @classmethod
    def from_device(cls, fmt: int, dev_blocks, n: int, k: int, n_mats: int = 1) -> "Weights":
        nb01 = formats.row_bytes(fmt, k)
        h = C.c_void_p()
        _check(load().fq_weights_from_device(fmt, _vp(dev_blocks), nb01, nb01 * n, n, k, n_mats, C.byref(h)))
        return cls(h.value, fmt, n, k, n_mats)

    def view(self, row0: int, rows: int) -> "Weights":
        """Rows [row0, row0 + rows) of every stacked matrix, without a copy (keep `self` alive while the view is used)."""
        h = C.c_void_p()
        _check(load().fq_weights_view(self.handle, row0, rows, C.byref(h)))
        v = Weights(h.value, self.fmt, rows, self.k, self.n_mats)
        v.parent = self
        return v

    def device_bytes(self) -> int:
        return int(load().fq_weights_device_bytes(self.handle))

    def download_gguf(self) -> np.ndarray:
        nb01 = formats.row_bytes(self.fmt, self.k)
        out = np.zeros((self.n_mats * self.n, nb01), dtype=np.uint8)
        _check(load().fq_weights_download_gguf(self.handle, _vp(out), out.size))
        return out

    def dequantize(self, mat: int = 0, row0: int = 0, rows: int | None = None) -> np.ndarray:
        rows = self.n - row0 if rows is None else rows
        out = np.zeros((rows, self.k), dtype=np.float32)
        _check(load().fq_dequantize_rows(self.handle, mat, row0, rows, _vp(out)))
        return out

    def free(self) -> None:
        if self.handle:
            load().fq_weights_free(self.handle)
            self.handle = 0

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


def attn_fwd(q: np.ndarray, k: np.ndarray, v: np.ndarray, kv_head_for_head, source_offset: int, scale: float, window: int = 0,
             causal: bool = True, want_stats: bool = False):
    """Twin of `attnPrefillF16` / the f32-KV forward (src/backend/cuda.zig:2601-2736): q [q_seq, heads, d] f32,
    k/v [kv_seq, kv_heads, d] f16 or f32 -> out [q_seq, heads, d] (and stats [heads, q_seq, 2])."""
    q = np.ascontiguousarray(q, dtype=np.float32)
    f16 = k.dtype == np.float16
    k = np.ascontiguousarray(k, dtype=np.float16 if f16 else np.float32)
    v = np.ascontiguousarray(v, dtype=k.dtype)
    q_seq, heads, d = q.shape
    kv_seq, kv_heads, _ = k.shape
    kvmap = np.ascontiguousarray(kv_head_for_head, dtype=np.int32)
    out = np.full_like(q, np.nan)
    stats = np.full((heads, q_seq, 2), np.nan, dtype=np.float32) if want_stats else None
    _check(load().fq_attn_fwd(_vp(q), _vp(k), _vp(v), int(f16), _vp(out), _vp(stats), _vp(kvmap), q_seq, kv_seq, heads, kv_heads, d,
                              source_offset, scale, window, int(causal)))
    return (out, stats) if want_stats else out


def attn_fwd_dev(q_dev, k_dev, v_dev, kv_is_f16: bool, out_dev, kvmap_dev, q_seq: int, kv_seq: int, heads: int, kv_heads: int, d: int,
                 source_offset: int, scale: float, window: int = 0, causal: bool = True, stats_dev=None, stream: int = 0) -> None:
    _check(load().fq_attn_fwd_dev(_vp(q_dev), _vp(k_dev), _vp(v_dev), int(kv_is_f16), _vp(out_dev), _vp(stats_dev), _vp(kvmap_dev), q_seq,
                                  kv_seq, heads, kv_heads, d, source_offset, scale, window, int(causal), C.c_void_p(stream)))


class _GgufTensor(C.Structure):
    _fields_ = [("name", C.c_char_p), ("ggml_type", C.c_int), ("fmt", C.c_int), ("n_dims", C.c_int), ("dims", C.c_uint64 * 4),
                ("offset", C.c_uint64), ("bytes", C.c_uint64)]


class Gguf:
    """A mapped GGUF file (`fq_gguf`): tensor table and metadata without a GPU, resident weights with one.

    Mirrors what the reference does with src/gguf.zig + the residency hooks of src/weights.zig:2621-2816."""

    def __init__(self, path: str):
        h = C.c_void_p()
        _check(load().fq_gguf_open(os.fsencode(path), C.byref(h)))
        self.handle = h.value

    def tensors(self) -> list[dict]:
        out = []
        for i in range(int(load().fq_gguf_tensor_count(self.handle))):
            t = _GgufTensor()
            _check(load().fq_gguf_tensor_at(self.handle, i, C.byref(t)))
            out.append({"name": t.name.decode("utf-8", "replace"), "ggml_type": t.ggml_type, "fmt": t.fmt, "dims": list(t.dims[: t.n_dims]),
                        "offset": int(t.offset), "bytes": int(t.bytes)})
        return out

    def find(self, name: str) -> int:
        return int(load().fq_gguf_find(self.handle, name.encode()))

    def data(self, index: int, nbytes: int) -> np.ndarray:
        p = load().fq_gguf_tensor_data(self.handle, index)
        return np.ctypeslib.as_array(C.cast(p, C.POINTER(C.c_uint8)), shape=(nbytes,)).copy()

    def meta_u64(self, key: str) -> int:
        v = C.c_uint64()
        _check(load().fq_gguf_meta_u64(self.handle, key.encode(), C.byref(v)))
        return int(v.value)

    def meta_str(self, key: str) -> str:
        buf = C.create_string_buffer(4096)
        _check(load().fq_gguf_meta_str(self.handle, key.encode(), buf, len(buf)))
        return buf.value.decode("utf-8", "replace")

    def load_weights(self, name: str, row0: int = 0, rows: int = 0, mat0: int = 0, mats: int = 0) -> Weights:
        i = self.find(name)
        if i < 0:
            raise KeyError(name)
        t = self.tensors()[i]
        h = C.c_void_p()
        _check(load().fq_gguf_load_weights(self.handle, i, row0, rows, mat0, mats, C.byref(h)))
        dims = t["dims"] + [1] * (3 - len(t["dims"]))
        return Weights(h.value, t["fmt"], rows or dims[1] - row0, dims[0], mats or dims[2] - mat0)

    def load_ptqtp_planes(self, base: str, row0: int = 0, rows: int = 0, mat0: int = 0, mats: int = 0) -> list[Weights]:
        arr = (C.c_void_p * 3)()
        n = C.c_int()
        _check(load().fq_gguf_load_ptqtp_planes(self.handle, base.encode(), row0, rows, mat0, mats, arr, C.byref(n)))
        t = self.tensors()[self.find(base + ".ptqtp0")]
        dims = t["dims"] + [1] * (3 - len(t["dims"]))
        return [Weights(arr[p], formats.TQ2_0, rows or dims[1] - row0, dims[0], mats or dims[2] - mat0) for p in range(n.value)]

    def close(self) -> None:
        if self.handle:
            load().fq_gguf_close(self.handle)
            self.handle = 0

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def shard_rows(n: int, n_ranks: int, rank: int, align: int = 32) -> tuple[int, int]:
    r0, rows = C.c_size_t(), C.c_size_t()
    _check(load().fq_gguf_shard_rows(n, n_ranks, rank, align, C.byref(r0), C.byref(rows)))
    return int(r0.value), int(rows.value)


def quantize_rows_dev(fmt: int, dev_src, n: int, k: int, dev_blocks) -> None:
    """Weight encoder on the device: f32 [n, k] in HBM -> raw GGUF blocks in HBM."""
    _check(load().fq_quantize_rows_dev(fmt, _vp(dev_src), n, k, _vp(dev_blocks)))


# --------------------------------------------------------------------------- dense, host buffers
def gemm_quant_nt(fmt: int, rhs: np.ndarray, a: np.ndarray, n: int, cacheable: bool = False,
                  nb01: int | None = None, out: np.ndarray | None = None) -> np.ndarray:
    """`gemmQuantNt` (src/backend/cuda.zig:2398-2435): c[m,n] = a[m,k] . dequant(rhs)^T."""
    assert rhs.dtype == np.uint8 and rhs.flags["C_CONTIGUOUS"]
    a = np.ascontiguousarray(a, dtype=np.float32)
    m, k = a.shape
    nb01 = formats.row_bytes(fmt, k) if nb01 is None else nb01
    c = np.full((m, n), np.nan, dtype=np.float32) if out is None else out
    _check(load().fq_gemm_quant_nt(fmt, _vp(rhs), rhs.size, int(cacheable), nb01, _vp(a), _vp(c), m, n, k))
    return c


def gemm_quant_nt_shared_a_batch(fmt: int, rhs: np.ndarray, a: np.ndarray, n: int, batch: int,
                                 cacheable: bool = False) -> np.ndarray:
    """`gemmQuantNtSharedABatch` (src/backend/cuda.zig:2441-2492): one input, `batch` stacked matrices."""
    a = np.ascontiguousarray(a, dtype=np.float32)
    m, k = a.shape
    nb01 = formats.row_bytes(fmt, k)
    c = np.full((batch * m, n), np.nan, dtype=np.float32)
    _check(load().fq_gemm_quant_nt_shared_a_batch(fmt, _vp(rhs), rhs.size, int(cacheable), nb01, nb01 * n, _vp(a),
                                                  _vp(c), batch, m, n, k))
    return c


class Work:
    """Completion token (`accelerator.Work`, src/accelerator.zig:22-133)."""

    def __init__(self, handle: int, out: np.ndarray | None):
        self.handle, self.out = handle, out

    def finish(self, copy_to_host: bool = True) -> None:
        _check(load().fq_work_finish(self.handle, int(copy_to_host)))

    def device_ptr(self) -> int:
        return int(load().fq_work_device_ptr(self.handle))

    def destroy(self) -> None:
        if self.handle:
            load().fq_work_destroy(self.handle)
            self.handle = 0


def gemm_quant_nt_async(fmt: int, rhs: np.ndarray, a: np.ndarray | None, n: int, m: int, k: int, batch: int = 1,
                        dep: Work | None = None, out: np.ndarray | None = None) -> Work:
    """`gemmQuantNtAsync` (src/backend/cuda.zig:2001-2175); rhs must be process-stable bytes."""
    nb01 = formats.row_bytes(fmt, k)
    if a is not None:
        a = np.ascontiguousarray(a, dtype=np.float32)
    c = np.full((batch * m, n), np.nan, dtype=np.float32) if out is None else out
    h = C.c_void_p()
    _check(load().fq_gemm_quant_nt_async(fmt, _vp(rhs), rhs.size, 1, nb01, nb01 * n, _vp(a),
                                         C.c_void_p(dep.handle if dep else 0), _vp(c), batch, m, n, k, C.byref(h)))
    return Work(h.value, c)


class PreparedGemmAsync:
    """`gemm_quant_nt_async` with its arguments converted once, for a caller that repeats the same product every
    step (a decode loop: same resident weights, same host activation and result storage). `submit()` queues the
    product and returns at once; `finish()` waits, leaves the result in `out` and releases the token
    (`gemmQuantNtAsync` + `Work.finish`, src/backend/cuda.zig:2001-2175, src/accelerator.zig:22-133). The object keeps
    the three arrays alive; it holds at most one product in flight."""

    __slots__ = ("_submit", "_finish", "_destroy", "_args", "_h", "_keep", "out")

    def __init__(self, fmt: int, rhs: np.ndarray, a: np.ndarray, n: int, m: int, k: int, batch: int = 1, out: np.ndarray | None = None):
        if a.dtype != np.float32 or not a.flags.c_contiguous or a.size != m * k:
            raise ValueError("activations must be a C-contiguous float32 array of m * k elements")
        if out is None:
            out = np.full((batch * m, n), np.nan, dtype=np.float32)
        if out.dtype != np.float32 or not out.flags.c_contiguous or out.size != batch * m * n:
            raise ValueError("out must be a C-contiguous float32 array of batch * m * n elements")
        lib = load()
        nb01 = formats.row_bytes(fmt, k)
        self._submit, self._finish, self._destroy = lib.fq_gemm_quant_nt_async, lib.fq_work_finish, lib.fq_work_destroy
        self._h = C.c_void_p()
        self._args = (fmt, C.c_void_p(rhs.ctypes.data), rhs.size, 1, nb01, nb01 * n, C.c_void_p(a.ctypes.data), C.c_void_p(0),
                      C.c_void_p(out.ctypes.data), batch, m, n, k, C.byref(self._h))
        self._keep = (rhs, a)
        self.out = out

    def submit(self) -> None:
        if self._h.value:
            raise RuntimeError("the previous submit was not finished")
        rc = self._submit(*self._args)
        if rc:
            _check(rc)

    def finish(self) -> np.ndarray:
        if not self._h.value:
            raise RuntimeError("nothing was submitted")
        rc = self._finish(self._h, 1)
        self._destroy(self._h)
        self._h.value = None
        if rc:
            _check(rc)
        return self.out


# --------------------------------------------------------------------------- dense, device buffers
def gemm_quant_nt_dev(w: Weights, a_dev, c_dev, m: int, mat: int = 0, mode: int = MODE_AUTO, stream: int = 0) -> None:
    _check(load().fq_gemm_quant_nt_dev(w.handle, mat, _vp(a_dev), _vp(c_dev), m, mode, C.c_void_p(stream)))


PRE_NONE, PRE_RMS_NORM_MUL, PRE_SPLIT_SWIGLU = 0, 1, 2


def gemm_quant_nt_pre_dev(w: Weights, pre_op: int, a_dev, c_dev, m: int, pre_w_dev=None, eps: float = 0.0, mat: int = 0,
                          mode: int = MODE_AUTO, stream: int = 0) -> None:
    """Product with a row operation fused in front of the activation quantiser (src/exec/quant_matmul.zig:480-757):
    PRE_RMS_NORM_MUL (a_dev [m][k], pre_w_dev [k], eps) or PRE_SPLIT_SWIGLU (a_dev [m][2k], gate | up)."""
    _check(load().fq_gemm_quant_nt_pre_dev(w.handle, mat, pre_op, _vp(a_dev), _vp(pre_w_dev) if pre_w_dev is not None else None,
                                           eps, _vp(c_dev), m, mode, C.c_void_p(stream)))


def act_prologue_dev(pre_op: int, a_dev, out_dev, m: int, k: int, pre_w_dev=None, eps: float = 0.0, stream: int = 0) -> None:
    """The row operation of `gemm_quant_nt_pre_dev` alone: out_dev [m][k] f32."""
    _check(load().fq_act_prologue_dev(pre_op, _vp(a_dev), _vp(pre_w_dev) if pre_w_dev is not None else None, eps, _vp(out_dev),
                                      m, k, C.c_void_p(stream)))


def gemm_quant_nt_dev_noalloc(w: Weights, a_dev, c_dev, m: int, mat: int = 0, stream: int = 0) -> None:
    """Small-batch product for callers that may not allocate device memory while serving.

    Same numbers as `gemm_quant_nt_dev(..., mode=MODE_INT8)` for m <= 16; the activation
    scratch is a fixed 512 KiB array inside the library, shared by all calls (order
    them on one stream). Declined when the activation records would not fit.
    """
    _check(load().fq_gemm_quant_nt_dev_noalloc(w.handle, mat, _vp(a_dev), _vp(c_dev), m, C.c_void_p(stream)))


def small_batch_max_rows(fmt: int, k: int) -> int:
    """Rows one launch of the small-batch integer kernel takes for this format and k (0: none fit)."""
    return int(load().fq_small_batch_max_rows(fmt, k))


def gemm_ptqtp_dev(planes: list[Weights], a_dev, c_dev, m: int, stream: int = 0) -> None:
    """K ternary planes summed per element in plane order (src/weights.zig:204-300)."""
    arr = (C.c_void_p * len(planes))(*[p.handle for p in planes])
    _check(load().fq_gemm_ptqtp_dev(arr, len(planes), _vp(a_dev), _vp(c_dev), m, C.c_void_p(stream)))


def quantize_acts_q8_k_dev(a_dev, m: int, k: int, dev_blocks) -> None:
    _check(load().fq_quantize_acts_q8_k_dev(_vp(a_dev), m, k, _vp(dev_blocks)))


def quantize_acts_q8_0_dev(a_dev, m: int, k: int, dev_blocks) -> None:
    _check(load().fq_quantize_acts_q8_0_dev(_vp(a_dev), m, k, _vp(dev_blocks)))


class Graph:
    """A captured sequence of *_dev calls on the library stream, replayed with one launch."""

    def __init__(self, handle: int):
        self.handle = handle

    def launch(self) -> None:
        _check(load().fq_graph_launch(self.handle))

    def destroy(self) -> None:
        if self.handle:
            load().fq_graph_destroy(self.handle)
            self.handle = 0


class capture:
    """`with capture() as cap: ...dev calls...` then `cap.graph.launch()`."""

    def __enter__(self):
        _check(load().fq_capture_begin())
        self.graph = None
        return self

    def __exit__(self, et, ev, tb):
        h = C.c_void_p()
        rc = load().fq_capture_end(C.byref(h))
        if et is None:
            _check(rc)
            self.graph = Graph(h.value)
        return False


# --------------------------------------------------------------------------- MoE
def qmoe_stage(in_floats: int, out_floats: int):
    """`qmoeStage` (src/backend/cuda.zig:2221): the provider's pinned in/out panels as numpy views."""
    pin, pout = C.c_void_p(), C.c_void_p()
    _check(load().fq_qmoe_stage(in_floats * 4, out_floats * 4, C.byref(pin), C.byref(pout)))
    a = np.ctypeslib.as_array(C.cast(pin, C.POINTER(C.c_float)), shape=(in_floats,))
    b = np.ctypeslib.as_array(C.cast(pout, C.POINTER(C.c_float)), shape=(out_floats,))
    return a, b


def gemm_q_grouped_nt(fmt: int, rhs: np.ndarray, n_out: int, k: int, tiles: list[tuple[int, int, int, int]],
                      cacheable: bool = False) -> None:
    """`gemmQGroupedNt` (src/backend/cuda.zig:2244-2333) over the staged panels; caller holds the qmoe lock."""
    nb01 = formats.row_bytes(fmt, k)
    arr = (QmmTile * len(tiles))(*[QmmTile(*t) for t in tiles])
    _check(load().fq_gemm_q_grouped_nt(fmt, _vp(rhs), rhs.size, int(cacheable), nb01, nb01 * n_out, n_out, k, arr,
                                       len(tiles)))


def moe_layer(gate: Weights, up: Weights, down: Weights, x: np.ndarray, selected: np.ndarray, weights: np.ndarray,
              gated_op: int = 0) -> np.ndarray:
    """Twin of `ExecContext.moeExpertFfn` / `moeExpertFfnBatch` (src/exec/moe.zig:1135-1298, :1865-2088)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    seq = x.shape[0]
    selected = np.ascontiguousarray(selected, dtype=np.int64).reshape(seq, -1)
    top_k = selected.shape[1]
    weights = np.ascontiguousarray(weights, dtype=np.float32).reshape(seq, top_k)
    out = np.full_like(x, np.nan)
    _check(load().fq_moe_layer(gate.handle, up.handle, down.handle, _vp(x), seq, top_k, _vp(selected), _vp(weights),
                               gated_op, _vp(out)))
    return out


def moe_layer_dev(gate: Weights, up: Weights, down: Weights, x_dev, seq: int, top_k: int, selected_dev, weights_dev,
                  out_dev, gated_op: int = 0, stream: int = 0) -> None:
    _check(load().fq_moe_layer_dev(gate.handle, up.handle, down.handle, _vp(x_dev), seq, top_k, _vp(selected_dev),
                                   _vp(weights_dev), gated_op, _vp(out_dev), C.c_void_p(stream)))


def moe_layer_ptqtp_dev(gate_planes: list[Weights], up_planes: list[Weights], down_planes: list[Weights], x_dev, seq: int, top_k: int,
                        selected_dev, weights_dev, out_dev, gated_op: int = 0, stream: int = 0) -> None:
    """The expert layer over multi-plane ternary experts (`MoePtqtpRhs`, src/exec/moe.zig:51-78): K TQ2_0 stacks per projection."""
    K = len(gate_planes)
    arr = lambda ws: (C.c_void_p * K)(*[w.handle for w in ws])  # noqa: E731
    _check(load().fq_moe_layer_ptqtp_dev(arr(gate_planes), arr(up_planes), arr(down_planes), K, _vp(x_dev), seq, top_k, _vp(selected_dev),
                                         _vp(weights_dev), gated_op, _vp(out_dev), C.c_void_p(stream)))


def moe_layer_stages_for_test(gate: Weights, up: Weights, down: Weights, x_dev, seq: int, top_k: int, selected_dev,
                              weights_dev, g_pairs_dev, down_pairs_dev, out_dev) -> None:
    """The layer's integer arm with g and the unweighted down rows copied out in pair order (test seam)."""
    _check(load().fq_moe_layer_stages_for_test(gate.handle, up.handle, down.handle, _vp(x_dev), seq, top_k,
                                               _vp(selected_dev), _vp(weights_dev), _vp(g_pairs_dev),
                                               _vp(down_pairs_dev), _vp(out_dev)))


def moe_layer_ep_dev(gate: Weights, up: Weights, down: Weights, x_dev, seq: int, top_k: int, selected_dev, weights_dev,
                     expert_base: int, partial_dev, gated_op: int = 0, stream: int = 0) -> None:
    """This shard's partial output of the layer: experts [expert_base, expert_base + E_local), global ids in
    `selected_dev`, pairs of other shards skipped."""
    _check(load().fq_moe_layer_ep_dev(gate.handle, up.handle, down.handle, _vp(x_dev), seq, top_k, _vp(selected_dev),
                                      _vp(weights_dev), expert_base, gated_op, _vp(partial_dev), C.c_void_p(stream)))


# --------------------------------------------------------------------------- several GPUs, one process each
EP_AUTO, EP_NCCL, EP_FUSED = 0, 1, 2


def tp_unique_id() -> bytes:
    """The 128-byte rendezvous id rank 0 makes; the host carries it to the other ranks."""
    buf = C.create_string_buffer(128)
    _check(load().fq_tp_unique_id(buf))
    return buf.raw


def tp_init(n_ranks: int, rank: int, unique_id: bytes, arena_bytes: int = 0) -> None:
    assert len(unique_id) == 128
    _check(load().fq_tp_init(n_ranks, rank, C.c_char_p(unique_id), arena_bytes))


def tp_init_torch(dist, arena_bytes: int = 0) -> None:
    """fq_tp_init with the id carried by an initialised torch.distributed group (any backend)."""
    rank, world = dist.get_rank(), dist.get_world_size()
    box = [tp_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(box, src=0)
    tp_init(world, rank, box[0], arena_bytes)


def tp_shutdown() -> None:
    _check(load().fq_tp_shutdown())


def tp_peer_access() -> bool:
    return bool(load().fq_tp_peer_access())


def gemm_quant_nt_tp(w_shard: Weights, a_dev, c_dev, m: int, mode: int = MODE_AUTO, stream: int = 0) -> None:
    """Column-sharded product + all-gather: c_dev [rank][m][n_shard] on every rank (collective)."""
    _check(load().fq_gemm_quant_nt_tp(w_shard.handle, _vp(a_dev), _vp(c_dev), m, mode, C.c_void_p(stream)))


def moe_layer_ep(gate: Weights, up: Weights, down: Weights, x_dev, seq: int, top_k: int, selected_dev, weights_dev, out_dev,
                 flags: int = EP_AUTO, gated_op: int = 0, stream: int = 0) -> None:
    """Expert-parallel MoE layer over the ranks of `tp_init` (collective): this rank's tokens in, this rank's tokens out."""
    _check(load().fq_moe_layer_ep(gate.handle, up.handle, down.handle, _vp(x_dev), seq, top_k, _vp(selected_dev), _vp(weights_dev),
                                  gated_op, _vp(out_dev), flags, C.c_void_p(stream)))


def ep_emulate_for_test(gates: list[Weights], ups: list[Weights], downs: list[Weights], xs: list, seq: int, top_k: int, sels: list,
                        wts: list, outs: list, arena_bytes: int, layers: int = 1) -> None:
    """`len(gates)` ranks of the fused expert-parallel layer emulated on one GPU (test seam)."""
    world = len(gates)

    def arr(items, ptr=lambda t: t.data_ptr()):
        return (C.c_void_p * world)(*[ptr(t) for t in items])

    h = lambda w: w.handle  # noqa: E731
    _check(load().fq_ep_emulate_for_test(world, arr(gates, h), arr(ups, h), arr(downs, h), arr(xs), seq, top_k, arr(sels), arr(wts),
                                         arr(outs), arena_bytes, layers))


def router_topk_dev(logits_dev, seq: int, n_expert: int, top_k: int, normalize: bool, selected_dev, weights_dev,
                    stream: int = 0) -> None:
    """`routerTopK` (src/exec/topk.zig:21-86) on the device."""
    _check(load().fq_router_topk_dev(_vp(logits_dev), seq, n_expert, top_k, int(normalize), _vp(selected_dev),
                                     _vp(weights_dev), C.c_void_p(stream)))


# --------------------------------------------------------------------------- gates
def should_use_gpu_dense_quant(fmt: int, work: int) -> bool:
    return bool(load().fq_should_use_gpu_dense_quant(fmt, work))


def should_use_gpu_dense_quant_packed(fmt: int, work: int) -> bool:
    return bool(load().fq_should_use_gpu_dense_quant_packed(fmt, work))


def should_use_gpu_quant_decode(fmt: int, m: int, n: int, k: int) -> bool:
    return bool(load().fq_should_use_gpu_quant_decode(fmt, m, n, k))


def should_use_gpu_qmoe(work: int) -> bool:
    return bool(load().fq_should_use_gpu_qmoe(work))


def qmoe_fill_acceptable(rows: int, n_tiles: int) -> bool:
    return bool(load().fq_qmoe_fill_acceptable(rows, n_tiles))
