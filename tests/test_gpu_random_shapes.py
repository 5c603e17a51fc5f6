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
