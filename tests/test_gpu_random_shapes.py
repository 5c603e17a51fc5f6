"""GPU parity, seeded random sweep: formats, batch sizes, row counts and depths drawn at random (fixed seeds), each
product run on the integer arm against the CPU-kernel oracle (1e-3) and, where the tensor arm serves the shape, on
the tensor arm against the bf16 oracle (1e-2), through the device-buffer entry; then the same weights through the
blocking host-buffer entry in automatic mode, whose result must meet the bound of the arm it chose. Shapes the
hand-picked cases of the other files do not name: odd multiples of four rows, one to 70 activation rows, depths of
one to eight blocks."""
import numpy as np
import pytest

import oracle
from parity import TOL_INT8, TOL_TENSOR, assert_close, make_weights, rel_err, rms_err

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


def _draw(seed):
    rng = np.random.default_rng(90_000 + seed)
    name = FMTS[int(rng.integers(len(FMTS)))]
    k = 256 * int(rng.integers(1, 9))
    n = 4 * int(rng.integers(1, 176))
    m = int(rng.choice([1, 1, 2, 3, 4, 5, 7, 8, 9, 12, 16, 17, 23, 31, 32, 33, 47, 64, 70]))
    return name, m, n, k


@pytest.mark.parametrize("seed", range(48))
def test_random_shape(P, torch, seed):
    name, m, n, k = _draw(seed)
    fmt = oracle.FORMATS[name]
    blocks = make_weights(name, n, k, seed=91_000 + seed)
    a = np.random.default_rng(92_000 + seed).standard_normal((m, k)).astype(np.float32)
    what = f"seed {seed}: {name} {m}x{n}x{k}"
    w = P.Weights.upload(fmt, blocks, n, k)
    ad = torch.from_numpy(a).cuda()
    arms = {}
    for mode, label in ((P.MODE_INT8, "int8"), (P.MODE_TENSOR, "tensor")):
        cd = torch.full((m, n), float("nan"), dtype=torch.float32, device="cuda")
        torch.cuda.synchronize()
        try:
            P.gemm_quant_nt_dev(w, ad, cd, m, mode=mode)
        except P.Declined:
            assert mode == P.MODE_TENSOR, f"{what}: the integer arm serves every shape"
            continue
        P.synchronize()
        arms[label] = cd.cpu().numpy()
    w.free()
    want_a = oracle.matmul(fmt, blocks, a)
    want_b = oracle.matmul_dequant_f64(fmt, blocks, a, round_bf16=True)
    assert_close(arms["int8"], want_a, TOL_INT8, what + " (int8)")
    if "tensor" in arms:
        assert_close(arms["tensor"], want_b, TOL_TENSOR, what + " (tensor)")
    # the host-buffer entry picks an arm by itself (transient weights, row-major): the bound of whichever arm it took
    got = P.gemm_quant_nt(fmt, blocks, a, n, cacheable=False)
    ea, eb = rel_err(got, want_a), rel_err(got, want_b)
    assert ea <= TOL_INT8 or eb <= TOL_TENSOR, f"{what}: automatic mode is {ea:.2e} from the int8 oracle and {eb:.2e} from the bf16 oracle"


def _draw_moe(seed):
    rng = np.random.default_rng(95_000 + seed)
    name = ["q4_k", "q5_k", "q6_k", "q8_0"][int(rng.integers(4))]
    hidden = 256 * int(rng.integers(1, 5))
    out_pe = 256 * int(rng.integers(1, 4))
    n_expert = int(rng.choice([2, 3, 4, 7, 8, 16, 33]))
    top_k = int(rng.integers(1, min(n_expert, 6) + 1))
    seq = int(rng.choice([1, 2, 3, 5, 8, 13, 21, 40, 77, 150]))
    gated_op = int(rng.integers(0, 5))
    # every third case gives the down tensor another format, as mixed K-quant files do (Q4_K gate/up with a Q6_K down)
    down = ["q6_k", "q8_0", "q5_k", "q4_k"][int(rng.integers(4))] if seed % 3 == 2 else name
    return name, down, hidden, out_pe, n_expert, top_k, seq, gated_op


@pytest.mark.parametrize("seed", range(32))
def test_random_moe_layer(P, seed):
    """The fused expert layer on drawn shapes (formats, expert counts that are not powers of two, top-k 1..6, one to 150
    tokens, the five gated ops, every third case with a down tensor of another format), once on the integer arm against
    the int8 oracle and once on the tensor arm against the bf16 oracle."""
    from fucina_b200._lib import load

    name, name_dn, hidden, out_pe, n_expert, top_k, seq, gated_op = _draw_moe(seed)
    fmt, fmt_dn = oracle.FORMATS[name], oracle.FORMATS[name_dn]
    what = f"seed {seed}: {name}/{name_dn} hidden {hidden} ffn {out_pe} experts {n_expert} top-{top_k} seq {seq} op {gated_op}"
    gate = make_weights(name, n_expert * out_pe, hidden, seed=96_000 + 3 * seed)
    up = make_weights(name, n_expert * out_pe, hidden, seed=96_001 + 3 * seed)
    down = make_weights(name_dn, n_expert * hidden, out_pe, seed=96_002 + 3 * seed)
    rng = np.random.default_rng(97_000 + seed)
    x = (rng.standard_normal((seq, hidden)) * (12 if gated_op in (2, 4) else 1)).astype(np.float32)
    sel, w = oracle.router_topk(rng.standard_normal((seq, n_expert)).astype(np.float32), top_k, True)
    wg = P.Weights.upload(fmt, gate, out_pe, hidden, n_expert)
    wu = P.Weights.upload(fmt, up, out_pe, hidden, n_expert)
    wd = P.Weights.upload(fmt_dn, down, hidden, out_pe, n_expert)
    try:
        for arm in (0, 1):
            load().fq_set_moe_tensor_for_test(arm)
            got = P.moe_layer(wg, wu, wd, x, sel, w, gated_op=gated_op)
            if arm:
                want = oracle.moe_ffn_bf16(fmt, gate, up, down, x, sel, w, n_expert, out_pe, gated_op=gated_op, fmt_down=fmt_dn)
                rms = float(np.sqrt(np.mean(want.astype(np.float64) ** 2)))
                err = float(np.max(np.abs(got - want))) / rms
                assert np.isfinite(got).all() and err <= 1e-2, f"{what} (tensor): {err:.2e} of the output RMS"
            else:
                want = oracle.moe_ffn(fmt, gate, up, down, x, sel, w, n_expert, out_pe, gated_op=gated_op, fmt_down=fmt_dn)
                # an ulp of difference between the device's and the oracle's expf / tanhf can move a requantised
                # intermediate by one int8 step (1.5e-3 of the output RMS per flip at these widths): the bound is on
                # the RMS of the difference and on its largest element, both relative to the output RMS
                rms, worst = rms_err(got, want)
                assert rms <= 1e-3 and worst <= 1e-2, f"{what} (int8): rms {rms:.2e}, worst {worst:.2e} of the output RMS"
    finally:
        load().fq_set_moe_tensor_for_test(-1)
        for h in (wg, wu, wd):
            h.free()


@pytest.mark.parametrize("seed", range(24))
def test_random_attention(P, seed):
    """Streaming attention on drawn shapes (rows, keys, head grouping, head size, window, causal or not, f16 or f32 KV)
    against the f64 oracle with the reference's own bound (src/backend/cuda.zig:3547-3552)."""
    from test_gpu_attention import attn_f64, check

    rng = np.random.default_rng(98_000 + seed)
    kv_heads = int(rng.choice([1, 2, 3, 4, 8]))
    group = int(rng.choice([1, 2, 3, 4, 5, 8]))
    heads = kv_heads * group
    d = 8 * int(rng.integers(1, 33))
    f16 = bool(rng.integers(2))
    if not f16:
        d = 4 * int(rng.integers(1, 65))
    q_seq = int(rng.choice([1, 1, 1, 2, 3, 7, 16, 40]))
    kv_seq = q_seq + int(rng.choice([0, 1, 31, 64, 129, 500, 1500, 4100]))
    causal = bool(rng.integers(4))  # one in four bidirectional
    window = int(rng.choice([0, 0, 16, 100, 1000])) if causal else 0
    q = rng.standard_normal((q_seq, heads, d)).astype(np.float32)
    k = rng.standard_normal((kv_seq, kv_heads, d)).astype(np.float16 if f16 else np.float32)
    v = rng.standard_normal((kv_seq, kv_heads, d)).astype(k.dtype)
    kvmap = rng.permutation(np.repeat(np.arange(kv_heads), group)).tolist() if seed % 2 else [h // group for h in range(heads)]
    scale = float(1.0 / np.sqrt(d))
    got, stats = P.attn_fwd(q, k, v, kvmap, kv_seq - q_seq, scale, window, causal, want_stats=True)
    want, want_stats = attn_f64(q, k, v, kvmap, kv_seq - q_seq, scale, window, causal)
    check(got, want)
    assert np.allclose(stats[..., 0], want_stats[..., 0], rtol=1e-5, atol=1e-5), f"seed {seed}: row maxima"
    assert np.allclose(stats[..., 1], want_stats[..., 1], rtol=2e-4), f"seed {seed}: sums of exponentials"


@pytest.mark.parametrize("seed", range(16))
def test_random_grouped_tables(P, seed):
    """The grouped entry over drawn tile tables in the reference's form {expert, group base, group rows, tile index}:
    experts in any order, empty experts left out, groups of 1 to 150 rows; each group against the oracle of the arm
    that serves its run length (tensor cores from 17 rows, the integer kernel below)."""
    from fucina_b200._lib import load

    rng = np.random.default_rng(99_000 + seed)
    name = ["q4_k", "q5_k", "q8_0", "q6_k"][int(rng.integers(4))]
    fmt = oracle.FORMATS[name]
    n_expert = int(rng.integers(1, 9))
    n_out = 4 * int(rng.integers(1, 80))
    k = 256 * int(rng.integers(1, 5))
    counts = [int(c) for c in rng.choice([0, 0, 1, 2, 5, 8, 16, 17, 31, 32, 33, 64, 65, 150], size=n_expert)]
    if sum(counts) == 0:
        counts[0] = 3
    order = rng.permutation(n_expert).tolist()
    blocks = make_weights(name, n_out * n_expert, k, seed=99_100 + seed)
    rows = sum(counts)
    a = rng.standard_normal((rows, k)).astype(np.float32)
    tiles, base, where = [], 0, {}
    for e in order:  # groups laid out in the drawn expert order
        if counts[e] == 0:
            continue
        where[e] = base
        tiles += [(e, base, counts[e], t) for t in range((counts[e] + 31) // 32)]
        base += counts[e]
    lib = load()
    lib.fq_qmoe_lock()
    try:
        pin, pout = P.qmoe_stage(rows * k, rows * n_out)
        pin[:] = a.reshape(-1)
        pout[:] = np.nan
        P.gemm_q_grouped_nt(fmt, blocks, n_out, k, tiles)
        got = np.array(pout).reshape(rows, n_out)
    finally:
        lib.fq_qmoe_unlock()
    for e, b in where.items():
        m = counts[e]
        w, x, y = blocks[e * n_out:(e + 1) * n_out], a[b:b + m], got[b:b + m]
        ea = rel_err(y, oracle.matmul(fmt, w, x))
        eb = rel_err(y, oracle.matmul_dequant_f64(fmt, w, x, round_bf16=True))
        assert (ea <= TOL_INT8) if m < 17 else (eb <= TOL_TENSOR or ea <= TOL_INT8), \
            f"seed {seed}: {name} expert {e} ({m} rows at {b}): {ea:.2e} from the int8 oracle, {eb:.2e} from the bf16 oracle"


@pytest.mark.parametrize("seed", range(12))
def test_random_ptqtp_planes(P, torch, seed):
    """One to three ternary planes summed per element in plane order (src/weights.zig:204-300) on drawn shapes."""
    rng = np.random.default_rng(99_500 + seed)
    planes = int(rng.integers(1, 4))
    k = 256 * int(rng.integers(1, 17))
    n = 4 * int(rng.integers(1, 130))
    m = int(rng.choice([1, 1, 2, 3, 4, 5, 8, 16, 33, 64]))
    ps = []
    for p in range(planes):
        trits = rng.integers(-1, 2, size=(n, k)).astype(np.int8)
        scales = np.abs(rng.standard_normal((n, k // 256)) * 0.02 / (p + 1)).astype(np.float32)
        ps.append(oracle.pack_ptqtp_plane(trits, scales))
    a = rng.standard_normal((m, k)).astype(np.float32)
    ws = [P.Weights.upload(oracle.FORMATS["tq2_0"], b, n, k) for b in ps]
    ad = torch.from_numpy(a).cuda()
    cd = torch.full((m, n), float("nan"), device="cuda")
    torch.cuda.synchronize()
    P.gemm_ptqtp_dev(ws, ad, cd, m)
    P.synchronize()
    got = cd.cpu().numpy()
    for w in ws:
        w.free()
    ea = rel_err(got, oracle.matmul_ptqtp(ps, a))
    want_b = sum(oracle.matmul_dequant_f64(oracle.FORMATS["tq2_0"], b, a, round_bf16=True) for b in ps)
    eb = rel_err(got, want_b)
    assert ea <= TOL_INT8 or eb <= TOL_TENSOR, f"seed {seed}: K={planes} {m}x{n}x{k}: {ea:.2e} from the int8 oracle, {eb:.2e} from the bf16 oracle"
