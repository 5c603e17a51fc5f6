"""ctypes loader for libfucina_b200.so with every C-ABI signature declared."""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
# FUCINA_B200_LIB points at another build of the same library (a diagnostic build, for instance)
LIB_PATH = os.environ.get("FUCINA_B200_LIB") or os.path.join(_HERE, "lib", "libfucina_b200.so")

c_size = C.c_size_t
c_void = C.c_void_p
c_int = C.c_int
c_u64 = C.c_uint64
P = C.POINTER


class QmmTile(C.Structure):
    """`QMMTile` of the reference (src/backend/cuda.zig:1503-1508)."""

    _fields_ = [("expert", C.c_int32), ("base_row", C.c_int32), ("m", C.c_int32), ("tile_m", C.c_int32)]


# name -> (restype, argtypes); mirrors include/fucina_b200.h one to one
SIGNATURES = {
    "fq_init": (c_int, [c_int]),
    "fq_device_count": (c_int, []),
    "fq_device_name": (C.c_char_p, []),
    "fq_sm_count": (c_int, []),
    "fq_last_error": (c_int, [C.c_char_p, c_size]),
    "fq_stream": (c_void, []),
    "fq_synchronize": (c_int, []),
    "fq_block_elems": (c_size, [c_int]),
    "fq_block_bytes": (c_size, [c_int]),
    "fq_row_bytes": (c_size, [c_int, c_size]),
    "fq_alloc_resident": (c_void, [c_size]),
    "fq_free_resident": (None, [c_void]),
    "fq_evict_resident": (c_int, [c_void]),
    "fq_resident_bytes": (c_size, []),
    "fq_host_register": (c_int, [c_void, c_size]),
    "fq_host_unregister": (c_int, [c_void]),
    "fq_set_vram_budget": (c_int, [c_size]),
    "fq_weights_upload": (c_int, [c_int, c_void, c_size, c_size, c_size, c_size, c_size, P(c_void)]),
    "fq_weights_from_device": (c_int, [c_int, c_void, c_size, c_size, c_size, c_size, c_size, P(c_void)]),
    "fq_weights_view": (c_int, [c_void, c_size, c_size, P(c_void)]),
    "fq_weights_free": (None, [c_void]),
    "fq_weights_device_bytes": (c_size, [c_void]),
    "fq_weights_download_gguf": (c_int, [c_void, c_void, c_size]),
    "fq_dequantize_rows": (c_int, [c_void, c_size, c_size, c_size, c_void]),
    "fq_dequantize_rows_dev": (c_int, [c_void, c_size, c_size, c_size, c_void]),
    "fq_quantize_rows_dev": (c_int, [c_int, c_void, c_size, c_size, c_void]),
    "fq_gemm_quant_nt": (c_int, [c_int, c_void, c_size, c_int, c_size, c_void, c_void, c_size, c_size, c_size]),
    "fq_gemm_quant_nt_shared_a_batch": (
        c_int, [c_int, c_void, c_size, c_int, c_size, c_size, c_void, c_void, c_size, c_size, c_size, c_size]),
    "fq_gemm_quant_nt_async": (
        c_int, [c_int, c_void, c_size, c_int, c_size, c_size, c_void, c_void, c_void, c_size, c_size, c_size, c_size,
                P(c_void)]),
    "fq_work_finish": (c_int, [c_void, c_int]),
    "fq_work_device_ptr": (C.c_size_t, [c_void]),
    "fq_work_destroy": (None, [c_void]),
    "fq_gemm_quant_nt_dev": (c_int, [c_void, c_size, c_void, c_void, c_size, c_int, c_void]),
    "fq_gemm_quant_nt_dev_noalloc": (c_int, [c_void, c_size, c_void, c_void, c_size, c_void]),
    "fq_gemm_quant_nt_pre_dev": (c_int, [c_void, c_size, c_int, c_void, c_void, C.c_float, c_void, c_size, c_int, c_void]),
    "fq_act_prologue_dev": (c_int, [c_int, c_void, c_void, C.c_float, c_void, c_size, c_size, c_void]),
    "fq_small_batch_max_rows": (c_int, [c_int, c_size]),
    "fq_gemm_ptqtp_dev": (c_int, [P(c_void), c_int, c_void, c_void, c_size, c_void]),
    "fq_quantize_acts_q8_k_dev": (c_int, [c_void, c_size, c_size, c_void]),
    "fq_quantize_acts_q8_0_dev": (c_int, [c_void, c_size, c_size, c_void]),
    "fq_capture_begin": (c_int, []),
    "fq_capture_end": (c_int, [P(c_void)]),
    "fq_graph_launch": (c_int, [c_void]),
    "fq_graph_destroy": (None, [c_void]),
    "fq_qmoe_lock": (None, []),
    "fq_qmoe_unlock": (None, []),
    "fq_qmoe_stage": (c_int, [c_size, c_size, P(c_void), P(c_void)]),
    "fq_gemm_q_grouped_nt": (c_int, [c_int, c_void, c_size, c_int, c_size, c_size, c_size, c_size, P(QmmTile), c_size]),
    "fq_set_grouped_tensor_for_test": (None, [c_int]),
    "fq_moe_layer": (c_int, [c_void, c_void, c_void, c_void, c_size, c_size, c_void, c_void, c_int, c_void]),
    "fq_moe_layer_dev": (c_int, [c_void, c_void, c_void, c_void, c_size, c_size, c_void, c_void, c_int, c_void, c_void]),
    "fq_moe_layer_ptqtp_dev": (c_int, [P(c_void), P(c_void), P(c_void), c_int, c_void, c_size, c_size, c_void, c_void, c_int, c_void, c_void]),
    "fq_moe_layer_ep_dev": (
        c_int, [c_void, c_void, c_void, c_void, c_size, c_size, c_void, c_void, c_int, c_int, c_void, c_void]),
    "fq_tp_unique_id": (c_int, [c_void]),
    "fq_tp_init": (c_int, [c_int, c_int, c_void, c_size]),
    "fq_tp_shutdown": (c_int, []),
    "fq_tp_ranks": (c_int, []),
    "fq_tp_rank": (c_int, []),
    "fq_tp_peer_access": (c_int, []),
    "fq_gemm_quant_nt_tp": (c_int, [c_void, c_void, c_void, c_size, c_int, c_void]),
    "fq_moe_layer_ep": (c_int, [c_void, c_void, c_void, c_void, c_size, c_size, c_void, c_void, c_int, c_void, c_int, c_void]),
    "fq_ep_emulate_for_test": (c_int, [c_int, P(c_void), P(c_void), P(c_void), P(c_void), c_size, c_size, P(c_void), P(c_void), P(c_void),
                                       c_size, c_int]),
    "fq_router_topk_dev": (c_int, [c_void, c_size, c_size, c_size, c_int, c_void, c_void, c_void]),
    "fq_should_use_gpu_dense_quant": (c_int, [c_int, c_u64]),
    "fq_should_use_gpu_dense_quant_packed": (c_int, [c_int, c_u64]),
    "fq_should_use_gpu_quant_decode": (c_int, [c_int, c_size, c_size, c_size]),
    "fq_should_use_gpu_qmoe": (c_int, [c_u64]),
    "fq_qmoe_fill_acceptable": (c_int, [c_size, c_size]),
    "fq_set_min_work_qmoe_for_test": (None, [c_u64]),
    "fq_set_decode_for_test": (None, [c_int]),
    "fq_set_moe_tensor_for_test": (None, [c_int]),
    "fq_set_group_grid_limit_for_test": (None, [c_int]),
    "fq_moe_layer_stages_for_test": (c_int, [c_void, c_void, c_void, c_void, c_size, c_size, c_void, c_void, c_void, c_void, c_void]),
    "fq_attn_fwd_dev": (c_int, [c_void, c_void, c_void, c_int, c_void, c_void, c_void, c_size, c_size, c_size, c_size, c_size, c_size,
                                C.c_float, c_size, c_int, c_void]),
    "fq_attn_fwd": (c_int, [c_void, c_void, c_void, c_int, c_void, c_void, c_void, c_size, c_size, c_size, c_size, c_size, c_size, C.c_float,
                            c_size, c_int]),
    "fq_gguf_open": (c_int, [C.c_char_p, P(c_void)]),
    "fq_gguf_close": (None, [c_void]),
    "fq_gguf_tensor_count": (c_size, [c_void]),
    "fq_gguf_tensor_at": (c_int, [c_void, c_size, c_void]),
    "fq_gguf_find": (c_int, [c_void, C.c_char_p]),
    "fq_gguf_tensor_data": (c_void, [c_void, c_size]),
    "fq_gguf_meta_u64": (c_int, [c_void, C.c_char_p, P(c_u64)]),
    "fq_gguf_meta_str": (c_int, [c_void, C.c_char_p, C.c_char_p, c_size]),
    "fq_gguf_load_weights": (c_int, [c_void, c_size, c_size, c_size, c_size, c_size, P(c_void)]),
    "fq_gguf_load_ptqtp_planes": (c_int, [c_void, C.c_char_p, c_size, c_size, c_size, c_size, P(c_void), P(c_int)]),
    "fq_gguf_shard_rows": (c_int, [c_size, c_int, c_int, c_size, P(c_size), P(c_size)]),
    "fq_selftest_bounded_wait": (c_int, [C.c_uint]),
    "fq_trace_enabled": (c_int, []),
    "fq_trace_reset": (None, []),
    "fq_trace_dump": (None, []),
    "fq_trace_counters": (None, [P(c_u64)]),
    "fq_trace_kernel_timing": (None, [c_int]),
    "fq_trace_kernel_times": (c_int, [P(C.c_double), P(c_u64)]),
}

_lib = None


def load() -> C.CDLL:
    """Load the library or raise: there is no fallback path."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m fucina_b200.build` "
                "(nvcc, sm_100a). fucina_b200 has no CPU fallback."
            )
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)  # AttributeError here means header and library disagree
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib
