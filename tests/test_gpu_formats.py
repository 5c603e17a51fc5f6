"""GPU parity, part 1: gpu_formats. Everything here is bit-exact work --
repacking, dequantisation, activation quantisation, weight encoders -- checked
through the C ABI against the pinned oracle and the reference's goldens."""
import numpy as np
import pytest

import oracle
from parity import bits_equal, make_weights

pytestmark = pytest.mark.gpu

FMTS = ["q8_0", "q4_k", "q5_k", "q6_k", "tq2_0", "tq2_0_folded", "q2_0"]


@pytest.fixture(scope="module")
def P():
    from fucina_b200 import provider

    provider.init(0)
    assert "B200" in provider.device_name() or provider.sm_count() > 0
    return provider


@pytest.fixture(scope="module")
def torch():
    import torch

    assert torch.cuda.is_available()
    return torch


@pytest.mark.parametrize("fmt_name", FMTS)
@pytest.mark.parametrize("n,k", [(5, 256), (68, 512), (33, 4096)])
def test_repack_round_trip_is_byte_exact(P, fmt_name, n, k):
    fmt = oracle.FORMATS[fmt_name]
    blocks = make_weights(fmt_name, n, k, seed=11)
    w = P.Weights.upload(fmt, blocks, n, k)
    assert np.array_equal(w.download_gguf(), blocks)
    w.free()


@pytest.mark.parametrize("fmt_name", FMTS)
def test_dequantized_weights_are_bit_exact(P, fmt_name):
    fmt = oracle.FORMATS[fmt_name]
    n, k = 37, 1024
    blocks = make_weights(fmt_name, n, k, seed=12)
    w = P.Weights.upload(fmt, blocks, n, k)
    assert bits_equal(w.dequantize(), oracle.dequantize_rows(fmt, blocks, k))
    # a row window
    assert bits_equal(w.dequantize(row0=5, rows=9), oracle.dequantize_rows(fmt, blocks[5:14], k))
    w.free()


def test_q8_0_short_rows(P):
    # Q8_0 rows need not be multiples of 256 elements (k % 32 == 0 is the rule)
    for k in (32, 64, 96, 288):
        blocks = make_weights("q8_0", 12, k, seed=13)
        w = P.Weights.upload(oracle.Q8_0, blocks, 12, k)
        assert np.array_equal(w.download_gguf(), blocks)
        assert bits_equal(w.dequantize(), oracle.dequantize_rows(oracle.Q8_0, blocks, k))
        w.free()


def test_dequant_matches_reference_goldens(P, goldens):
    # ggml-produced blocks stored by the reference's tests
    w4 = P.Weights.upload(oracle.Q4_K, goldens["q4_k_golden"], 8, 256)
    assert bits_equal(w4.dequantize(), oracle.dequantize_rows(oracle.Q4_K, goldens["q4_k_golden"], 256))
    w5 = P.Weights.upload(oracle.Q5_K, goldens["q5_k_golden"], 8, 256)
    assert bits_equal(w5.dequantize(), oracle.dequantize_rows(oracle.Q5_K, goldens["q5_k_golden"], 256))
    w6 = P.Weights.upload(oracle.Q6_K, goldens["q6_k_golden"], 8, 256)
    assert bits_equal(w6.dequantize(), oracle.dequantize_rows(oracle.Q6_K, goldens["q6_k_golden"], 256))
    w6.free()
    tq = goldens["tq2_0_bytes"]
    wt = P.Weights.upload(oracle.TQ2_0, tq, tq.shape[0], 256)
    assert np.array_equal(wt.dequantize().view(np.uint32), goldens["tq2_0_expected_bits"])
    for w in (w4, w5, wt):
        w.free()


def test_expert_stack_layout(P):
    n, k, e = 8, 512, 5
    blocks = make_weights("q5_k", n * e, k, seed=14)
    w = P.Weights.upload(oracle.Q5_K, blocks, n, k, n_mats=e)
    for mat in range(e):
        assert bits_equal(w.dequantize(mat=mat), oracle.dequantize_rows(oracle.Q5_K, blocks[mat * n:(mat + 1) * n], k))
    w.free()


def _dev_encode(P, torch, fmt, x):
    n, k = x.shape
    xd = torch.from_numpy(x).cuda()
    out = torch.zeros(n * oracle.row_bytes(fmt, k), dtype=torch.uint8, device="cuda")
    P.quantize_rows_dev(fmt, xd, n, k, out)
    P.synchronize()
    return out.cpu().numpy().reshape(n, -1)


def test_weight_encoders_reproduce_ggml_goldens(P, torch, goldens):
    x = goldens["input_bits"].view(np.float32)
    assert np.array_equal(_dev_encode(P, torch, oracle.Q4_K, x), goldens["q4_k_golden"])
    assert np.array_equal(_dev_encode(P, torch, oracle.Q5_K, x), goldens["q5_k_golden"])
    assert np.array_equal(_dev_encode(P, torch, oracle.Q6_K, x), goldens["q6_k_golden"])


@pytest.mark.parametrize("fmt_name", ["q8_0", "q4_k", "q5_k", "q6_k", "tq2_0", "q2_0"])
def test_weight_encoders_match_oracle_bytes(P, torch, fmt_name):
    fmt = oracle.FORMATS[fmt_name]
    rng = np.random.default_rng(15)
    x = (rng.standard_normal((19, 1024)) * 0.02).astype(np.float32)
    x[3, 256:512] = 0.0  # an all-zero block
    x[4, :32] = 0.0
    assert np.array_equal(_dev_encode(P, torch, fmt, x), oracle.quantize_rows(fmt, x))


def test_q8_0_known_answers_on_device(P, torch):
    # src/backend/quant/q8_0_tests.zig:37-82
    src = (np.arange(32) - 16).astype(np.float32)
    src[0], src[31] = -127, 127
    got = _dev_encode(P, torch, oracle.Q8_0, src.reshape(1, 32))
    want_qs = (np.arange(32) - 16).astype(np.int8)
    want_qs[0], want_qs[31] = -127, 127
    assert int(got[0, :2].view(np.uint16)[0]) == int(np.array([1.0], np.float16).view(np.uint16)[0])
    assert np.array_equal(got[0, 2:].view(np.int8), want_qs)
    ties = np.zeros(32, np.float32)
    ties[:7] = [127, 0.5, 1.5, 2.5, -0.5, -1.5, -2.5]
    q = _dev_encode(P, torch, oracle.Q8_0, ties.reshape(1, 32))[0, 2:].view(np.int8)
    assert list(q[1:7]) == [1, 2, 3, -1, -2, -3]


@pytest.mark.parametrize("m,k", [(1, 256), (3, 4096), (16, 768), (5, 2048)])
def test_activation_quantisers_are_bit_exact(P, torch, m, k):
    rng = np.random.default_rng(16)
    a = rng.standard_normal((m, k)).astype(np.float32)
    a[0, :256] = 0.0                       # zero block: d = 0, all zeros
    if m > 1:
        a[1, 7] = a[1, 300 % k] = 9.5      # repeated maximum: the first one sets the scale
        a[1, 8] = -9.5
    ad = torch.from_numpy(a).cuda()
    out = torch.zeros(m * (k // 256) * 292, dtype=torch.uint8, device="cuda")
    P.quantize_acts_q8_k_dev(ad, m, k, out)
    P.synchronize()
    assert np.array_equal(out.cpu().numpy().reshape(m, -1), oracle.quantize_acts_q8_k(a))
    out0 = torch.zeros(m * (k // 32) * 34, dtype=torch.uint8, device="cuda")
    P.quantize_acts_q8_0_dev(ad, m, k, out0)
    P.synchronize()
    assert np.array_equal(out0.cpu().numpy().reshape(m, -1), oracle.quantize_acts_q8_0(a))


def test_q8_k_ties_round_to_even(P, torch):
    # inv*v lands exactly on .5: round-half-even, unlike the Q8_0 encoder
    a = np.zeros((1, 256), np.float32)
    a[0, 0] = -127.0  # inv = 1.0
    a[0, 1:7] = [0.5, 1.5, 2.5, -0.5, -1.5, -2.5]
    ad = torch.from_numpy(a).cuda()
    out = torch.zeros(292, dtype=torch.uint8, device="cuda")
    P.quantize_acts_q8_k_dev(ad, 1, 256, out)
    P.synchronize()
    got = out.cpu().numpy()
    assert np.array_equal(got.reshape(1, -1), oracle.quantize_acts_q8_k(a))
    assert list(got[4:11].view(np.int8)) == [-127, 0, 2, 2, 0, -2, -2]
