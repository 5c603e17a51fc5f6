"""The allocation-free entry point (collected last on purpose).

Servers that hand all of their VRAM to weights and KV cache at start-up, or that
cannot tolerate the device-wide stall of a cudaMalloc inside the decode loop,
call `fq_gemm_quant_nt_dev_noalloc`: its activation scratch is a fixed array in
the library image. It must give the same numbers as the regular device entry
point, call after call, even though every call reuses the same scratch.
"""
import numpy as np
import pytest

import oracle
from parity import TOL_INT8, assert_close, make_weights

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def P():
    from fucina_b200 import provider

    provider.init(0)
    return provider


@pytest.fixture(scope="module")
def torch():
    import torch

    return torch


def _both(P, torch, w, a, n):
    m = a.shape[0]
    ad = torch.from_numpy(a).cuda()
    ref = torch.full((m, n), float("nan"), dtype=torch.float32, device="cuda")
    got = torch.full((m, n), float("nan"), dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    P.gemm_quant_nt_dev(w, ad, ref, m, mode=P.MODE_INT8)
    P.gemm_quant_nt_dev_noalloc(w, ad, got, m)
    P.synchronize()
    return got.cpu().numpy(), ref.cpu().numpy()


@pytest.mark.parametrize("fmt_name,n,k", [("q4_k", 4096, 4096), ("q5_k", 132, 768), ("q8_0", 68, 160), ("tq2_0", 96, 1024)])
def test_matches_regular_entry_on_two_calls_in_a_row(P, torch, fmt_name, n, k):
    fmt = oracle.FORMATS[fmt_name]
    blocks = make_weights(fmt_name, n, k, seed=31)
    w = P.Weights.upload(fmt, blocks, n, k)
    rng = np.random.default_rng(32)
    # two different problems back to back: the second call finds the first one's records in the
    # shared scratch and must not be affected by them (more rows first, then fewer)
    for m in (5, 2):
        a = rng.standard_normal((m, k)).astype(np.float32)
        got, ref = _both(P, torch, w, a, n)
        assert_close(got, ref, TOL_INT8, f"{fmt_name} m={m} vs regular entry")
        assert_close(got, oracle.matmul(fmt, blocks, a), TOL_INT8, f"{fmt_name} m={m} vs oracle")
    w.free()


def test_same_kernel_means_same_bits(P, torch):
    # for a shape the regular entry also serves with the lane-per-chunk kernel the results are identical
    n, k, m = 100, 512, 9
    blocks = make_weights("q4_k", n, k, seed=33)
    w = P.Weights.upload(oracle.Q4_K, blocks, n, k)
    a = np.random.default_rng(34).standard_normal((m, k)).astype(np.float32)
    for _ in range(2):
        got, ref = _both(P, torch, w, a, n)
        assert np.array_equal(got.view(np.uint32), ref.view(np.uint32))
    w.free()


def test_sizes_beyond_the_fixed_scratch_are_declined(P, torch):
    n, k = 64, 65536  # 16 rows of about 1.4*k bytes do not fit in 512 KiB
    blocks = make_weights("q8_0", n, k, seed=35)
    w = P.Weights.upload(oracle.Q8_0, blocks, n, k)
    a = torch.zeros((16, k), dtype=torch.float32, device="cuda")
    c = torch.full((16, n), 7.0, dtype=torch.float32, device="cuda")
    with pytest.raises(P.Declined) as e:
        P.gemm_quant_nt_dev_noalloc(w, a, c, 16)
    assert "scratch" in str(e.value)
    with pytest.raises(P.Declined):
        P.gemm_quant_nt_dev_noalloc(w, a, c, 17)  # more rows than one pass takes
    P.synchronize()
    assert float(c.min()) == 7.0  # nothing was written
    w.free()


def test_rows_that_fit_the_array_but_not_shared_memory_are_declined(P, torch):
    # 16 rows of k = 16384 (Q8_0) are 352 KiB of records -- inside the 512 KiB array -- but the kernel keeps
    # them in shared memory, which holds 227 KiB: declined before anything is launched or written
    n, k = 64, 16384
    assert 8 <= P.small_batch_max_rows(oracle.Q8_0, k) < 16
    blocks = make_weights("q8_0", n, k, seed=36)
    w = P.Weights.upload(oracle.Q8_0, blocks, n, k)
    a = np.random.default_rng(37).standard_normal((16, k)).astype(np.float32)
    ad = torch.from_numpy(a).cuda()
    c = torch.full((16, n), 7.0, dtype=torch.float32, device="cuda")
    with pytest.raises(P.Declined) as e:
        P.gemm_quant_nt_dev_noalloc(w, ad, c, 16)
    assert e.value.code == 1 and "shared memory" in str(e.value)
    P.synchronize()
    assert float(c.min()) == 7.0 and float(c.max()) == 7.0
    # eight rows fit both bounds and still give the regular entry's numbers
    got, ref = _both(P, torch, w, a[:8], n)
    assert_close(got, ref, TOL_INT8, "m=8 after the decline")
    w.free()
