"""GPU parity, part 4: the bf16 tensor-core (tcgen05) prefill path against Oracle B --
an f64 dot over the oracle-dequantised weights with both operands rounded to bf16,
the reference's own GPU-test oracle (src/backend/cuda.zig:3016-3044) at this
build's operand precision. Tolerance: max relative error 1e-2, as the target states."""
import numpy as np
import pytest

import oracle
from parity import TOL_TENSOR, assert_close, make_weights

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


def run_tensor(P, torch, fmt, blocks, a, n, mode=None):
    m, k = a.shape
    w = P.Weights.upload(fmt, blocks, n, k)
    ad = torch.from_numpy(a).cuda()
    cd = torch.full((m, n), float("nan"), dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    P.gemm_quant_nt_dev(w, ad, cd, m, mode=P.MODE_TENSOR if mode is None else mode)
    P.synchronize()
    w.free()
    return cd.cpu().numpy()


@pytest.mark.parametrize("fmt_name", ["q4_k", "q5_k", "q6_k", "q8_0", "tq2_0", "tq2_0_folded", "q2_0"])
@pytest.mark.parametrize("m,n,k", [
    (64, 128, 256),      # one tile, one block of K
    (33, 96, 512),       # the reference's ragged parity shape (cuda.zig:3084-3088): partial rows and tokens
    (300, 388, 1024),    # two token tiles, four row tiles, ragged on both sides
    (512, 1024, 4096),   # prefill width
])
def test_tensor_path_matches_bf16_oracle(P, torch, fmt_name, m, n, k):
    fmt = oracle.FORMATS[fmt_name]
    blocks = make_weights(fmt_name, n, k, seed=2000 + n)
    a = np.random.default_rng(2100 + m).standard_normal((m, k)).astype(np.float32)
    got = run_tensor(P, torch, fmt, blocks, a, n)
    want = oracle.matmul_dequant_f64(fmt, blocks, a, round_bf16=True)
    err = assert_close(got, want, TOL_TENSOR, f"{fmt_name} {m}x{n}x{k}")
    assert err < 1e-3  # f32 accumulation over identical bf16 operands is far inside the bound


def test_auto_mode_routes_large_m_to_tensor_cores(P, torch):
    n, k, m = 256, 1024, 96
    blocks = make_weights("q4_k", n, k, seed=2200)
    a = np.random.default_rng(2201).standard_normal((m, k)).astype(np.float32)
    auto = run_tensor(P, torch, oracle.Q4_K, blocks, a, n, mode=P.MODE_AUTO)
    tens = run_tensor(P, torch, oracle.Q4_K, blocks, a, n)
    assert np.array_equal(auto.view(np.uint32), tens.view(np.uint32))
    # and it stays close to the CPU kernels' int8 result (information: activation quantisation noise,
    # measured at matrix level because near-zero outputs have no meaningful relative error)
    want = oracle.matmul(oracle.Q4_K, blocks, a)
    assert float(np.max(np.abs(tens - want)) / np.max(np.abs(want))) < 5e-2


@pytest.mark.parametrize("fmt_name,hidden,out_pe,n_expert,top_k,seq", [
    ("q5_k", 256, 256, 4, 2, 37),      # ragged expert runs inside one 128-token tile: fused gate/up pass, SwiGLU in the epilogue
    ("q5_k", 512, 768, 8, 4, 300),     # runs of ~150 rows, several row tiles, Qwen3-MoE expert width
    ("q4_k", 256, 512, 4, 2, 700),     # runs longer than one 256-token tile
    ("q8_0", 256, 256, 4, 2, 60),      # split rows read by the dequantising threads, fused gate/up pass on 128-token tiles
    ("q8_0", 256, 256, 2, 2, 300),     # the same format on 256-token tiles (separate gate and up products)
])
def test_moe_tensor_arm_matches_bf16_oracle(P, fmt_name, hidden, out_pe, n_expert, top_k, seq):
    from fucina_b200._lib import load

    fmt = oracle.FORMATS[fmt_name]
    rng = np.random.default_rng(2400)
    gate = make_weights(fmt_name, n_expert * out_pe, hidden, 2401)
    up = make_weights(fmt_name, n_expert * out_pe, hidden, 2402)
    down = make_weights(fmt_name, n_expert * hidden, out_pe, 2403)
    x = rng.standard_normal((seq, hidden)).astype(np.float32)
    sel, w = oracle.router_topk(rng.standard_normal((seq, n_expert)).astype(np.float32), top_k, True)
    wg = P.Weights.upload(fmt, gate, out_pe, hidden, n_expert)
    wu = P.Weights.upload(fmt, up, out_pe, hidden, n_expert)
    wd = P.Weights.upload(fmt, down, hidden, out_pe, n_expert)
    load().fq_set_moe_tensor_for_test(1)
    try:
        got = P.moe_layer(wg, wu, wd, x, sel, w)
    finally:
        load().fq_set_moe_tensor_for_test(-1)
    want = oracle.moe_ffn_bf16(fmt, gate, up, down, x, sel, w, n_expert, out_pe)
    # The layer rounds the intermediate g to bf16. Kernel and oracle compute g with different
    # accumulation (f32 tensor core vs f64), so a few g values land on the other side of a bf16
    # rounding boundary; one such flip moves an output by ~3e-4 of the output RMS, which the
    # per-element ratio would blow up on near-zero outputs. The bound is therefore on the error
    # relative to the output scale: 1e-2 of the RMS (observed ~1e-3).
    rms = float(np.sqrt(np.mean(want.astype(np.float64) ** 2)))
    err = float(np.max(np.abs(got - want))) / rms
    assert np.isfinite(got).all() and err <= TOL_TENSOR, f"moe tensor arm {fmt_name} seq={seq}: {err:.3e} of output RMS"
    # the two arms agree to activation-quantisation noise (matrix level)
    int8 = oracle.moe_ffn(fmt, gate, up, down, x, sel, w, n_expert, out_pe)
    assert float(np.max(np.abs(got - int8)) / np.max(np.abs(int8))) < 5e-2
    for h in (wg, wu, wd):
        h.free()


def test_shapes_without_a_tensor_kernel_are_declined_in_tensor_mode(P, torch):
    n, k, m = 64, 288, 32   # Q8_0 rows of nine 32-weight blocks: fine for the integer kernels, not a whole number of K slabs
    blocks = make_weights("q8_0", n, k, seed=2300)
    a = np.zeros((m, k), np.float32)
    with pytest.raises(P.Declined):
        run_tensor(P, torch, oracle.Q8_0, blocks, a, n)
    # AUTO falls back to the integer kernel in 16-row passes
    got = run_tensor(P, torch, oracle.Q8_0, blocks, a + 1.0, n, mode=P.MODE_AUTO)
    assert_close(got, oracle.matmul(oracle.Q8_0, blocks, a + 1.0), 1e-3, "q8_0 auto")


@pytest.mark.parametrize("planes", [1, 2])
def test_ptqtp_planes_on_the_tensor_cores(P, torch, planes):
    """A prefill-sized multi-plane ternary product: every plane is a tensor-core product over bf16-rounded
    operands, the planes are added per element in plane order (src/weights.zig:286-300)."""
    n, k, m = 192, 1024, 100
    rng = np.random.default_rng(2500 + planes)
    ps = []
    for p in range(planes):
        trits = rng.integers(-1, 2, size=(n, k)).astype(np.int8)
        scales = np.abs(rng.standard_normal((n, k // 256)) * 0.02 / (3 ** p)).astype(np.float32)
        ps.append(oracle.pack_ptqtp_plane(trits, scales))
    a = rng.standard_normal((m, k)).astype(np.float32)
    ws = [P.Weights.upload(oracle.TQ2_0, b, n, k) for b in ps]
    ad = torch.from_numpy(a).cuda()
    cd = torch.full((m, n), float("nan"), dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    P.gemm_ptqtp_dev(ws, ad, cd, m)
    P.synchronize()
    want = sum(oracle.matmul_dequant_f64(oracle.TQ2_0, b, a, round_bf16=True) for b in ps)
    assert_close(cd.cpu().numpy(), want, TOL_TENSOR, f"ptqtp tensor K={planes}")
    for w in ws:
        w.free()


@pytest.mark.parametrize("fmt_name", ["q4_k", "q8_0"])
@pytest.mark.parametrize("m,n,k", [(200, 150 * 128, 1024), (300, 75 * 128 + 40, 2048)])
def test_split_k_tail_of_a_partly_filled_last_wave(P, torch, fmt_name, m, n, k):
    # more tiles than SMs with a last wave that fills at most half of them: its tiles are cut along K and the parts
    # added in order by a second kernel (150 tiles = 148 + 2; 2 x 76 = 152 = 148 + 4, ragged rows and tokens)
    from parity import oracle_b

    fmt = oracle.FORMATS[fmt_name]
    blocks = make_weights(fmt_name, n, k, seed=2300 + m)
    a = np.random.default_rng(2301 + m).standard_normal((m, k)).astype(np.float32)
    got = run_tensor(P, torch, fmt, blocks, a, n)
    err = assert_close(got, oracle_b(fmt, blocks, a, k), TOL_TENSOR, f"{fmt_name} {m}x{n}x{k}")
    assert err < 1e-3
    assert not np.isnan(got).any()
