"""GPU parity, part 2: quantized matmul through the C ABI against Oracle A
(the CPU-kernel replica: int8 activations, integer block dots, f32 epilogue).
Tolerance: max relative error 1e-3 (f32 accumulate), as the target states."""
import numpy as np
import pytest

import oracle
from parity import TOL_INT8, assert_close, make_weights

pytestmark = pytest.mark.gpu

FMTS = ["q8_0", "q4_k", "q5_k", "q6_k", "tq2_0", "tq2_0_folded", "q2_0"]


@pytest.fixture(scope="module")
def P():
    from fucina_b200 import provider

    provider.init(0)
    return provider


@pytest.fixture(scope="module")
def torch():
    import torch

    return torch


def acts(m, k, seed):
    return np.random.default_rng(seed).standard_normal((m, k)).astype(np.float32)


def run_dev(P, torch, fmt, blocks, a, n, mode=None):
    m, k = a.shape
    w = P.Weights.upload(fmt, blocks, n, k)
    ad = torch.from_numpy(a).cuda()
    cd = torch.full((m, n), float("nan"), dtype=torch.float32, device="cuda")
    P.gemm_quant_nt_dev(w, ad, cd, m, mode=P.MODE_INT8 if mode is None else mode)
    P.synchronize()
    w.free()
    return cd.cpu().numpy()


# the reference's own GPU parity shapes (src/backend/cuda.zig:3084-3088, :3307-3312)
# with B = 256 (32 for Q8_0), plus decode widths
def ref_shapes(fmt_name):
    B = 32 if fmt_name == "q8_0" else 256
    return [(1, 68, 2 * B), (4, 68, 2 * B), (3, 68, 2 * B), (16, 96, B), (2, 64, 2 * B)]


@pytest.mark.parametrize("fmt_name", FMTS)
def test_reference_parity_shapes(P, torch, fmt_name):
    fmt = oracle.FORMATS[fmt_name]
    for (m, n, k) in ref_shapes(fmt_name):
        blocks = make_weights(fmt_name, n, k, seed=100 + m)
        a = acts(m, k, 200 + m)
        got = run_dev(P, torch, fmt, blocks, a, n)
        assert_close(got, oracle.matmul(fmt, blocks, a), TOL_INT8, f"{fmt_name} {m}x{n}x{k}")


@pytest.mark.parametrize("fmt_name", FMTS)
@pytest.mark.parametrize("m", [1, 2, 3, 4, 5, 8, 9, 16])
def test_decode_batches(P, torch, fmt_name, m):
    fmt = oracle.FORMATS[fmt_name]
    n, k = 132, 2048
    blocks = make_weights(fmt_name, n, k, seed=300)
    a = acts(m, k, 400 + m)
    got = run_dev(P, torch, fmt, blocks, a, n)
    assert_close(got, oracle.matmul(fmt, blocks, a), TOL_INT8, f"{fmt_name} m={m}")


@pytest.mark.parametrize("fmt_name", FMTS)
@pytest.mark.parametrize("k", [256, 768, 1280, 4096, 11008 - 11008 % 256])
def test_row_lengths_and_lane_groupings(P, torch, fmt_name, k):
    # 768 and 1280 exercise the 8- and 16-lane row groups, 4096 the full-warp one
    fmt = oracle.FORMATS[fmt_name]
    n, m = 52, 2
    blocks = make_weights(fmt_name, n, k, seed=500)
    a = acts(m, k, 600)
    got = run_dev(P, torch, fmt, blocks, a, n)
    assert_close(got, oracle.matmul(fmt, blocks, a), TOL_INT8, f"{fmt_name} k={k}")


def test_q8_0_rows_shorter_than_a_superblock(P, torch):
    for k in (32, 64, 160):
        blocks = make_weights("q8_0", 68, k, seed=700)
        a = acts(3, k, 701)
        got = run_dev(P, torch, oracle.Q8_0, blocks, a, 68)
        assert_close(got, oracle.matmul(oracle.Q8_0, blocks, a), TOL_INT8, f"q8_0 k={k}")


@pytest.mark.parametrize("fmt_name", ["q8_0", "q4_k", "q5_k", "tq2_0"])
def test_committed_oracle_fixture(P, torch, oracle_cases, fmt_name):
    fmt = oracle.FORMATS[fmt_name]
    blocks, a, want = oracle_cases[f"{fmt_name}_blocks"], oracle_cases[f"{fmt_name}_a"], oracle_cases[f"{fmt_name}_matmul"]
    got = run_dev(P, torch, fmt, blocks, a, blocks.shape[0])
    assert_close(got, want, TOL_INT8, fmt_name)


@pytest.mark.parametrize("fmt_name", ["q4_k", "q8_0"])
@pytest.mark.parametrize("m", [17, 33, 64])
def test_more_rows_than_one_pass_int8(P, torch, fmt_name, m):
    fmt = oracle.FORMATS[fmt_name]
    n, k = 96, 512
    blocks = make_weights(fmt_name, n, k, seed=800)
    a = acts(m, k, 801)
    got = run_dev(P, torch, fmt, blocks, a, n)
    assert_close(got, oracle.matmul(fmt, blocks, a), TOL_INT8, f"{fmt_name} m={m}")


def test_saturating_activations_and_zero_rows(P, torch):
    # every activation at the block maximum (all quantise to +-127) and an all-zero row
    k, n = 512, 68
    blocks = make_weights("q4_k", n, k, seed=900)
    a = np.ones((3, k), np.float32) * 7.25
    a[1] *= -1
    a[2] = 0
    got = run_dev(P, torch, oracle.Q4_K, blocks, a, n)
    want = oracle.matmul(oracle.Q4_K, blocks, a)
    assert_close(got[:2], want[:2], TOL_INT8, "saturated")
    assert np.array_equal(got[2], np.zeros(n, np.float32))


@pytest.mark.parametrize("planes", [1, 2, 3])
def test_ptqtp_plane_sum(P, torch, planes):
    # K planes summed per element in plane order (src/weights.zig:286-300)
    n, k, m = 68, 1024, 2
    rng = np.random.default_rng(1000)
    ps = []
    for p in range(planes):
        trits = rng.integers(-1, 2, size=(n, k)).astype(np.int8)
        scales = np.abs(rng.standard_normal((n, k // 256)) * 0.02 / (3**p)).astype(np.float32)
        ps.append(oracle.pack_ptqtp_plane(trits, scales))
    a = acts(m, k, 1001)
    ws = [P.Weights.upload(oracle.TQ2_0, b, n, k) for b in ps]
    ad = torch.from_numpy(a).cuda()
    cd = torch.full((m, n), float("nan"), dtype=torch.float32, device="cuda")
    P.gemm_ptqtp_dev(ws, ad, cd, m)
    P.synchronize()
    assert_close(cd.cpu().numpy(), oracle.matmul_ptqtp(ps, a), TOL_INT8, f"ptqtp K={planes}")
    for w in ws:
        w.free()


def test_row_permutation_equivariance_at_full_size(P, torch):
    # size-independent property at the decode stack's largest shape: every output
    # row depends on its own weight row only, so reversing the weight rows
    # reverses the outputs bit for bit
    n, k = 32000, 4096
    rng = np.random.default_rng(1100)
    blocks = np.tile(rng.integers(0, 256, size=(n, 144), dtype=np.uint8), (1, k // 256))
    half = np.array([0.01], np.float16).view(np.uint8)
    blocks.reshape(n, k // 256, 144)[:, :, 0:2] = half
    blocks.reshape(n, k // 256, 144)[:, :, 2:4] = half
    a = acts(1, k, 1101)
    y = run_dev(P, torch, oracle.Q4_K, blocks, a, n)
    y_rev = run_dev(P, torch, oracle.Q4_K, np.ascontiguousarray(blocks[::-1]), a, n)
    assert np.array_equal(y.view(np.uint32), y_rev[:, ::-1].view(np.uint32))
    # and the values themselves, on a slice the oracle finishes quickly
    want = oracle.matmul(oracle.Q4_K, blocks[:2048], a)
    assert_close(y[:, :2048], want, TOL_INT8, "lm_head slice")


def test_full_size_decode_against_oracle(P, torch):
    # the Q8_0 bench shape (bench/q8gemv.zig: n = k = 4096, m = 1)
    n = k = 4096
    blocks = make_weights("q8_0", n, k, seed=1200)
    a = acts(1, k, 1201)
    got = run_dev(P, torch, oracle.Q8_0, blocks, a, n)
    assert_close(got, oracle.matmul(oracle.Q8_0, blocks, a), TOL_INT8, "q8gemv shape")


@pytest.mark.parametrize("fmt_name", ["q4_k", "q5_k", "q6_k", "q8_0"])
@pytest.mark.parametrize("n,k", [(64, 2048), (100, 2304), (333, 4096), (1000, 11008), (4096, 4096)])
def test_dense_decode_kernel_shapes(P, torch, fmt_name, n, k):
    # shapes the TMA-staged row-per-lane kernel takes: ragged row tiles (n not a
    # multiple of 32), ragged K slabs (9 and 43 blocks per row), more CTAs than row tiles
    fmt = oracle.FORMATS[fmt_name]
    blocks = make_weights(fmt_name, n, k, seed=1400 + n)
    for m in (1, 2, 3, 5, 8):
        a = acts(m, k, 1500 + m)
        got = run_dev(P, torch, fmt, blocks, a, n)
        assert_close(got, oracle.matmul(fmt, blocks, a), TOL_INT8, f"{fmt_name} {m}x{n}x{k}")


def test_dense_decode_is_deterministic(P, torch):
    n, k = 4096, 4096
    blocks = make_weights("q4_k", n, k, seed=1600)
    a = acts(1, k, 1601)
    y1 = run_dev(P, torch, oracle.Q4_K, blocks, a, n)
    y2 = run_dev(P, torch, oracle.Q4_K, blocks, a, n)
    assert np.array_equal(y1.view(np.uint32), y2.view(np.uint32))


def test_int8_path_stays_near_the_dequantised_product(P, torch):
    # Oracle B (f64 over dequantised weights, exact f32 activations): the int8
    # activation quantisation moves outputs by well under 5% of the output RMS.
    n, k = 256, 4096
    blocks = make_weights("q4_k", n, k, seed=1300)
    a = acts(2, k, 1301)
    got = run_dev(P, torch, oracle.Q4_K, blocks, a, n)
    want = oracle.matmul_dequant_f64(oracle.Q4_K, blocks, a)
    rms = float(np.sqrt(np.mean(want**2)))
    assert float(np.max(np.abs(got - want))) < 0.05 * rms


@pytest.mark.parametrize("m", [1, 2, 3, 4])
@pytest.mark.parametrize("n,k", [(64, 2048), (100, 2560), (1000, 4096), (8192, 8192), (4747, 3072)])
def test_ternary_planes_in_the_copy_engine_decode_kernel(P, torch, m, n, k):
    # TQ2_0 rows with k % 512 == 0 and up to four activation rows stream through the TMA-staged decode kernel
    # (16 warps from k = 8192); ragged row counts, more tiles than SMs, 8- and 16-warp forms
    blocks = make_weights("tq2_0", n, k, seed=1300 + n)
    a = acts(m, k, 1301 + m)
    got = run_dev(P, torch, oracle.TQ2_0, blocks, a, n)
    sl = slice(0, min(n, 1024))   # the scalar oracle on a slice of the largest shapes
    assert_close(got[:, sl], oracle.matmul(oracle.TQ2_0, blocks[sl], a), TOL_INT8, f"tq2_0 decode {m}x{n}x{k}")
    if n > 1024:
        tail = slice(n - 300, n)
        assert_close(got[:, tail], oracle.matmul(oracle.TQ2_0, blocks[tail], a), TOL_INT8, f"tq2_0 decode tail {m}x{n}x{k}")
    assert not np.isnan(got).any()


@pytest.mark.parametrize("planes", [2, 3])
def test_ptqtp_plane_sum_at_decode_width(P, torch, planes):
    # the planes of one product accumulate in launch order inside the decode kernel (k = 4096 takes that kernel)
    n, k, m = 300, 4096, 2
    rng = np.random.default_rng(1400)
    ps = []
    for p in range(planes):
        trits = rng.integers(-1, 2, size=(n, k)).astype(np.int8)
        scales = np.abs(rng.standard_normal((n, k // 256)) * 0.02 / (3**p)).astype(np.float32)
        ps.append(oracle.pack_ptqtp_plane(trits, scales))
    a = acts(m, k, 1401)
    ws = [P.Weights.upload(oracle.TQ2_0, b, n, k) for b in ps]
    ad = torch.from_numpy(a).cuda()
    cd = torch.full((m, n), float("nan"), dtype=torch.float32, device="cuda")
    P.gemm_ptqtp_dev(ws, ad, cd, m)
    P.synchronize()
    assert_close(cd.cpu().numpy(), oracle.matmul_ptqtp(ps, a), TOL_INT8, f"ptqtp K={planes} k={k}")
    for w in ws:
        w.free()
