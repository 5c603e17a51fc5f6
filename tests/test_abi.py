"""CPU-side checks of the C-ABI library: it loads, exports every symbol the
header declares, and the entry points that need no device behave."""
import ctypes as C
import os
import re

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from fucina_b200 import build

    build.build()
    from fucina_b200._lib import load

    return load()


def header_functions():
    text = open(os.path.join(ROOT, "include", "fucina_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(fq_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_a_real_surface():
    names = header_functions()
    assert len(names) >= 45
    for must in ("fq_gemm_quant_nt", "fq_gemm_quant_nt_async", "fq_gemm_q_grouped_nt", "fq_alloc_resident",
                 "fq_free_resident", "fq_moe_layer", "fq_work_finish", "fq_should_use_gpu_dense_quant"):
        assert must in names


def test_library_exports_every_declared_symbol(lib):
    for name in header_functions():
        assert hasattr(lib, name), f"{name} declared in include/fucina_b200.h but not exported"


def test_binding_table_matches_header():
    from fucina_b200._lib import SIGNATURES

    assert sorted(SIGNATURES) == header_functions()


def test_block_geometry(lib):
    from fucina_b200 import formats as F

    for fmt, (elems, nbytes) in F.BLOCK.items():
        assert lib.fq_block_elems(fmt) == elems
        assert lib.fq_block_bytes(fmt) == nbytes
        assert lib.fq_row_bytes(fmt, elems * 8) == nbytes * 8
        assert F.row_bytes(fmt, elems * 8) == nbytes * 8
    assert lib.fq_block_elems(4) == 0 and lib.fq_block_elems(15) == 0  # ids outside the enum are declined everywhere
    # the sizes the reference asserts (src/dtype.zig:230-239)
    assert (F.BLOCK[F.Q8_0], F.BLOCK[F.Q4_K], F.BLOCK[F.Q5_K], F.BLOCK[F.TQ2_0]) == ((32, 34), (256, 144), (256, 176), (256, 66))


def test_gates_keep_the_reference_predicates_with_b200_floors(lib):
    # the predicates of src/backend/cuda.zig:2494-2554 with the work floors measured on B200 (the reference's
    # defaults, :118-159, are the crossovers of a laptop GPU): blocking host-buffer call against the all-core CPU arm
    from fucina_b200 import formats as F

    assert lib.fq_should_use_gpu_qmoe(1 << 24) == 1
    assert lib.fq_should_use_gpu_qmoe((1 << 24) - 1) == 0
    for fmt in (F.Q4_K, F.Q5_K, F.Q8_0):
        assert lib.fq_should_use_gpu_dense_quant_packed(fmt, 1 << 22) == 1
        assert lib.fq_should_use_gpu_dense_quant_packed(fmt, (1 << 22) - 1) == 0
        assert lib.fq_should_use_gpu_dense_quant(fmt, 1 << 22) == 1
        assert lib.fq_should_use_gpu_dense_quant(fmt, (1 << 22) - 1) == 0
    assert lib.fq_should_use_gpu_dense_quant(F.Q6_K, 1 << 22) == 1
    assert lib.fq_should_use_gpu_dense_quant(7, 1 << 40) == 0  # not a format
    # a 7B-class prefill product and the decode stack's smallest product pass; the reference's defaults declined both
    assert lib.fq_should_use_gpu_dense_quant(F.Q4_K, 32 * 4096 * 4096) == 1
    assert lib.fq_should_use_gpu_quant_decode(F.Q5_K, 1, 4096, 4096) == 1
    # fill gate: rows*100 >= tiles*32*50
    assert lib.fq_qmoe_fill_acceptable(16, 1) == 1
    assert lib.fq_qmoe_fill_acceptable(15, 1) == 0
    assert lib.fq_qmoe_fill_acceptable(10, 0) == 0
    # decode gate: m*n*k >= 2^22 for every format (a 25 us call does not pay for less against the packed CPU arms)
    assert lib.fq_should_use_gpu_quant_decode(F.Q4_K, 1, 2048, 2048) == 1
    assert lib.fq_should_use_gpu_quant_decode(F.Q4_K, 1, 1024, 2048) == 0
    assert lib.fq_should_use_gpu_quant_decode(F.Q4_K, 1, 64, 256) == 0
    assert lib.fq_should_use_gpu_quant_decode(F.Q5_K, 1, 1024, 1024) == 0
    assert lib.fq_should_use_gpu_quant_decode(F.Q5_K, 4, 1024, 1024) == 1
    assert lib.fq_should_use_gpu_quant_decode(F.Q8_0, 1, 4096, 1024) == 1
    lib.fq_set_decode_for_test(0)
    assert lib.fq_should_use_gpu_quant_decode(F.Q4_K, 1, 4096, 4096) == 0
    lib.fq_set_decode_for_test(1)
    lib.fq_set_min_work_qmoe_for_test(1)
    assert lib.fq_should_use_gpu_qmoe(1) == 1
    lib.fq_set_min_work_qmoe_for_test(1 << 24)


def test_argument_rules_decline_before_touching_a_device(lib):
    # n % 4 != 0, k not a whole number of blocks, unknown format: the reference
    # returns false for each (src/backend/cuda.zig:2014-2022)
    from fucina_b200 import formats as F
    from fucina_b200 import provider as P

    a = np.zeros((1, 256), np.float32)
    rhs = np.zeros((8, 144), np.uint8)
    with pytest.raises(P.Declined) as e:
        P.gemm_quant_nt(F.Q4_K, rhs[:7], a, n=7)
    assert e.value.code == 1
    with pytest.raises(P.Declined) as e:
        P.gemm_quant_nt(7, rhs, a, n=8, nb01=210)
    assert e.value.code == 1
    with pytest.raises(P.Declined):
        P.gemm_quant_nt(F.Q4_K, rhs, np.zeros((1, 128), np.float32), n=8, nb01=144)


def test_no_gpu_means_decline_not_fallback(lib):
    import torch

    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    from fucina_b200 import formats as F
    from fucina_b200 import provider as P

    a = np.ones((1, 256), np.float32)
    rhs = np.zeros((8, 144), np.uint8)
    with pytest.raises(P.Declined) as e:
        P.gemm_quant_nt(F.Q4_K, rhs, a, n=8)
    assert e.value.code == 2  # FQ_DECLINED_NO_GPU
    assert lib.fq_alloc_resident(1024) is None


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    import fucina_b200._lib as L

    monkeypatch.setattr(L, "_lib", None)
    monkeypatch.setattr(L, "LIB_PATH", str(tmp_path / "nope.so"))
    with pytest.raises(ImportError):
        L.load()


def test_small_batch_row_limit_follows_shared_memory(lib):
    # the small-batch kernel keeps pad(m) activation records in <= 227 KiB of shared memory
    from fucina_b200 import formats as F

    def record(fmt, k):
        chunk, act_block = {F.Q8_0: (16, 32), F.Q4_K: (32, 256), F.Q5_K: (32, 256), F.TQ2_0: (64, 256),
                            F.TQ2_0_FOLDED: (32, 256), F.Q2_0: (64, 32)}[fmt]
        pad16 = lambda v: (v + 15) & ~15
        return k + pad16(k // chunk * 4) + pad16(k // act_block * 4)

    for fmt in (F.Q8_0, F.Q4_K, F.Q5_K, F.TQ2_0, F.TQ2_0_FOLDED, F.Q2_0):
        for k in (256, 4096, 11008 - 11008 % 256, 14336, 16384, 28672, 65536, 262144):
            want = next((mb for mb in (16, 8, 4, 2, 1) if mb * record(fmt, k) <= 227 * 1024), 0)
            assert lib.fq_small_batch_max_rows(fmt, k) == want, (fmt, k)
    assert lib.fq_small_batch_max_rows(F.Q4_K, 4096) == 16
    assert lib.fq_small_batch_max_rows(F.Q4_K, 28672) == 4       # the window the shared-memory rule closes
    assert lib.fq_small_batch_max_rows(F.Q8_0, 16384) == 8
    assert lib.fq_small_batch_max_rows(F.Q4_K, 262144) == 0
    assert lib.fq_small_batch_max_rows(7, 4096) == 0             # not a format
    assert lib.fq_small_batch_max_rows(F.Q4_K, 100) == 0         # not a whole number of blocks
