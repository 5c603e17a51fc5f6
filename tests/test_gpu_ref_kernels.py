"""GPU parity, cross-check: this library against the reference's own CUDA kernels
(src/backend/cuda/kernels.cu compiled unmodified for sm_100a into oracle/_ref by
oracle/build.py) on the same device buffers, the way the reference's GPU tests compare
its kernels with a dequantised product (src/backend/cuda.zig:3016-3044, :3291-3340).

The reference kernels dequantise to f32 (decode) or f16 (tiles) and keep f32 / f16
activations; this library follows the reference's CPU kernels (int8 activations) on the
decode arm and multiplies bf16 operands on the tensor arm. The two therefore differ by
operand-rounding noise that scales with the output's RMS, not with each element: measured
on the CPU oracles for these shapes, int8 activations move a product by 0.5-0.7 % of the
output RMS (largest element 2.4 %), bf16 operands by 0.23-0.26 % (largest 0.9 %). Each test
checks three sides: the reference kernel against the exact f64 product of the dequantised
weights, this library against its own oracle at the target's tolerance, and the two GPU
results against each other inside those noise bounds. Skipped where the reference checkout
was not present at build time."""
import numpy as np
import pytest

import oracle
from oracle import ref_cuda
from parity import TOL_INT8, TOL_TENSOR, assert_close, make_weights, rms_err

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not ref_cuda.available(), reason="oracle/_ref/libref_cuda.so was not built")]

FMTS = ["q8_0", "q6_k", "q4_k", "q5_k"]


@pytest.fixture(scope="module")
def P():
    from fucina_b200 import provider

    provider.init(0)
    return provider


@pytest.fixture(scope="module")
def torch():
    import torch

    return torch


def _raw(torch, blocks):
    return torch.from_numpy(np.ascontiguousarray(blocks).view(np.uint8).reshape(-1)).cuda()


@pytest.mark.parametrize("fmt_name", FMTS)
@pytest.mark.parametrize("m", [1, 3, 8])
def test_decode_arm_against_reference_gemv(P, torch, fmt_name, m):
    fmt, n, k = oracle.FORMATS[fmt_name], 256, 1024
    assert ref_cuda.FORMATS[fmt_name] == fmt
    blocks = make_weights(fmt_name, n, k, seed=7000 + m)
    a = np.random.default_rng(7100 + m).standard_normal((m, k)).astype(np.float32)
    raw, ad = _raw(torch, blocks), torch.from_numpy(a).cuda()
    ref = torch.full((m, n), float("nan"), device="cuda")
    torch.cuda.synchronize()
    ref_cuda.gemv(fmt, raw.data_ptr(), ad.data_ptr(), ref.data_ptr(), k, n, m, raw.numel() // n)
    torch.cuda.synchronize()
    ref = ref.cpu().numpy()
    # the reference kernel itself against the f64 product of the oracle-dequantised weights: f32 summation noise only
    assert_close(ref, oracle.matmul_dequant_f64(fmt, blocks, a), 1e-4, f"reference gemv {fmt_name} m={m}")
    got = P.gemm_quant_nt(fmt, blocks, a, n, cacheable=False)
    assert_close(got, oracle.matmul(fmt, blocks, a), TOL_INT8, f"{fmt_name} m={m} against the CPU-kernel oracle")
    rms, worst = rms_err(got, ref)
    assert rms <= 1e-2 and worst <= 5e-2, f"{fmt_name} m={m} against the reference gemv: rms {rms:.2e}, worst {worst:.2e} of the output RMS"


@pytest.mark.parametrize("fmt_name", FMTS)
@pytest.mark.parametrize("m,n,k", [(96, 192, 1024), (33, 96, 512)])
def test_tensor_arm_against_reference_tiles(P, torch, fmt_name, m, n, k):
    fmt = oracle.FORMATS[fmt_name]
    blocks = make_weights(fmt_name, n, k, seed=7200 + n)
    a = np.random.default_rng(7300 + m).standard_normal((m, k)).astype(np.float32)
    raw, ad = _raw(torch, blocks), torch.from_numpy(a).cuda()
    tiles = torch.tensor(ref_cuda.dense_tiles(m), dtype=torch.int32, device="cuda")
    nb01 = raw.numel() // n
    for n_tile, split_k in ((64, 1), (32, 1), (64, 2)):
        ref = torch.full((m, n), float("nan"), device="cuda")
        part = torch.empty((split_k, m, n), device="cuda")
        torch.cuda.synchronize()
        ref_cuda.mul_mm(fmt, raw.data_ptr(), ad.data_ptr(), tiles.data_ptr(), tiles.shape[0], ref.data_ptr(), k, n, nb01, nb01 * n,
                        part.data_ptr(), split_k, m * n, n_tile)
        torch.cuda.synchronize()
        refh = ref.cpu().numpy()
        # f16 operands in the reference kernel: 2^-12 relative rounding per operand
        rms, worst = rms_err(refh, oracle.matmul_dequant_f64(fmt, blocks, a))
        assert rms <= 1e-3 and worst <= 5e-3, f"reference tiles {fmt_name} N{n_tile} split {split_k}: rms {rms:.2e}, worst {worst:.2e}"
        w = P.Weights.upload(fmt, blocks, n, k)
        cd = torch.full((m, n), float("nan"), device="cuda")
        torch.cuda.synchronize()
        P.gemm_quant_nt_dev(w, ad, cd, m, mode=P.MODE_TENSOR)
        P.synchronize()
        w.free()
        got = cd.cpu().numpy()
        assert_close(got, oracle.matmul_dequant_f64(fmt, blocks, a, round_bf16=True), TOL_TENSOR, f"{fmt_name} {m}x{n}x{k} against the bf16 oracle")
        rms, worst = rms_err(got, refh)
        assert rms <= 4e-3 and worst <= 2e-2, f"{fmt_name} {m}x{n}x{k} against the reference tiles: rms {rms:.2e}, worst {worst:.2e}"


def test_grouped_tiles_against_reference(P, torch):
    """Expert-grouped product over the reference's tile table {expert, base_row, m, tile_m}: its kernel and
    fq_gemm_q_grouped_nt on the same table (the reference's own tile case 1, 7, 33, 40 rows)."""
    fmt, E, n, k = oracle.FORMATS["q5_k"], 4, 128, 512
    counts = [1, 7, 33, 40]
    rows = sum(counts)
    blocks = make_weights("q5_k", E * n, k, seed=7400)
    a = np.random.default_rng(7401).standard_normal((rows, k)).astype(np.float32)
    raw, ad = _raw(torch, blocks), torch.from_numpy(a).cuda()
    table = ref_cuda.grouped_tiles(counts)
    tiles = torch.tensor(table, dtype=torch.int32, device="cuda")
    nb01 = raw.numel() // (E * n)
    ref = torch.full((rows, n), float("nan"), device="cuda")
    torch.cuda.synchronize()
    ref_cuda.mul_mm(fmt, raw.data_ptr(), ad.data_ptr(), tiles.data_ptr(), len(table), ref.data_ptr(), k, n, nb01, nb01 * n)
    torch.cuda.synchronize()
    from fucina_b200._lib import load

    lib = load()
    lib.fq_qmoe_lock()
    try:
        pin, pout = P.qmoe_stage(rows * k, rows * n)
        pin[:] = a.reshape(-1)
        pout[:] = np.nan
        P.gemm_q_grouped_nt(fmt, blocks, n, k, [tuple(t) for t in table])  # the very table the reference kernel took
        got = np.array(pout).reshape(rows, n)
    finally:
        lib.fq_qmoe_unlock()
    # runs of 1 and 7 rows multiply on the integer kernel, those of 33 and 40 rows on the tensor cores
    rms, worst = rms_err(got, ref.cpu().numpy())
    assert rms <= 1e-2 and worst <= 5e-2, f"grouped q5_k against the reference tiles: rms {rms:.2e}, worst {worst:.2e}"


@pytest.mark.parametrize("q_seq,kv_seq,heads,kv_heads,d,window,causal,f16", [
    (64, 64, 8, 4, 64, 0, True, True),       # the reference's prefill cases (src/backend/cuda.zig:3484-3556)
    (33, 97, 4, 4, 48, 0, True, True),
    (40, 40, 8, 2, 128, 16, True, True),
    (37, 37, 6, 3, 80, 0, False, True),
    (1, 4099, 32, 8, 128, 0, True, True),    # a decode step: splits merged by this library's second kernel
    (2, 777, 8, 2, 64, 0, True, False),      # f32 KV
])
def test_attention_against_reference_kernel(P, torch, q_seq, kv_seq, heads, kv_heads, d, window, causal, f16):
    g = torch.Generator(device="cuda").manual_seed(7500 + kv_seq)
    q = torch.randn((q_seq, heads, d), generator=g, device="cuda")
    kv_t = torch.float16 if f16 else torch.float32
    k = torch.randn((kv_seq, kv_heads, d), generator=g, device="cuda").to(kv_t)
    v = torch.randn((kv_seq, kv_heads, d), generator=g, device="cuda").to(kv_t)
    kvmap = torch.tensor([h * kv_heads // heads for h in range(heads)], dtype=torch.int32, device="cuda")
    offset, scale = kv_seq - q_seq, float(1.0 / np.sqrt(d))
    ref, got = (torch.full_like(q, float("nan")) for _ in range(2))
    ref_s, got_s = (torch.full((heads, q_seq, 2), float("nan"), device="cuda") for _ in range(2))
    torch.cuda.synchronize()
    ref_cuda.attn_fwd(f16, q.data_ptr(), k.data_ptr(), v.data_ptr(), ref.data_ptr(), ref_s.data_ptr(), kvmap.data_ptr(), q_seq, kv_seq, heads,
                      kv_heads, d, offset, scale, window, causal)
    torch.cuda.synchronize()
    P.attn_fwd_dev(q, k, v, f16, got, kvmap, q_seq, kv_seq, heads, kv_heads, d, offset, scale, window, causal, stats_dev=got_s)
    P.synchronize()
    ref, got, ref_s, got_s = (t.cpu().numpy().astype(np.float64) for t in (ref, got, ref_s, got_s))
    # the reference's own bound for this kernel against its f64 oracle (cuda.zig:3547-3552), here between the two kernels
    tol = np.maximum(2e-3 * np.maximum(np.abs(ref), np.abs(got)), 2e-3)
    assert np.isfinite(got).all() and np.all(np.abs(got - ref) <= tol), float(np.max(np.abs(got - ref)))
    # {row max, sum of exponentials}: the same pair up to f32 rounding of the scores
    assert np.allclose(got_s[..., 0], ref_s[..., 0], rtol=0, atol=2e-3)
    assert np.allclose(got_s[..., 1], ref_s[..., 1], rtol=4e-3, atol=0)
