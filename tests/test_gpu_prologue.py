"""GPU parity: the row operations fused in front of the activation quantiser (RMSNorm * weight, split SwiGLU),
the reference's CPU fusions of src/exec/quant_matmul.zig:480-757, through the C ABI.

Three stages, so that every tolerance is explained: (1) the row operation alone against the oracle's scalar law at
f32 round-off; (2) the fused product against the stand-alone operation followed by the plain product, bit for bit
(the reference states the same property for its own fusion, src/exec/row_ops.zig:36-39); (3) the fused product
against the oracle's integer product fed the device's own activations at the 1e-3 of every other int8 product."""
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

    assert torch.cuda.is_available()
    return torch


def _inputs(op, m, k, seed):
    rng = np.random.default_rng(seed)
    if op == 1:
        x = (rng.standard_normal((m, k)) * 1.7).astype(np.float32)
        w = (1.0 + 0.1 * rng.standard_normal(k)).astype(np.float32)
        return x, w, 1e-6
    return rng.standard_normal((m, 2 * k)).astype(np.float32), None, 0.0


def _oracle_pre(op, x, w, eps):
    return oracle.rms_norm_mul(x, w, eps) if op == 1 else oracle.split_swiglu(x)


def _dev_pre(P, torch, op, x, w, eps, k):
    m = x.shape[0]
    xd = torch.from_numpy(x).cuda()
    wd = torch.from_numpy(w).cuda() if w is not None else None
    out = torch.full((m, k), float("nan"), dtype=torch.float32, device="cuda")
    P.act_prologue_dev(op, xd, out, m, k, pre_w_dev=wd, eps=eps)
    P.synchronize()
    return out


@pytest.mark.parametrize("op", [1, 2])
@pytest.mark.parametrize("m,k", [(1, 256), (3, 4096), (5, 11008 - 11008 % 256), (64, 2048)])
def test_row_operation_matches_the_scalar_law(P, torch, op, m, k):
    x, w, eps = _inputs(op, m, k, 7000 + m)
    got = _dev_pre(P, torch, op, x, w, eps, k).cpu().numpy()
    want = _oracle_pre(op, x, w, eps)
    # f32 round-off only: the sum of squares is added in another order (relative 1e-7 on the scale), exp differs by an ulp
    assert float(np.max(np.abs(got - want) / np.maximum(np.abs(want), 1e-6))) < 4e-6


@pytest.mark.parametrize("fmt_name", ["q4_k", "q5_k", "q8_0", "q6_k"])
@pytest.mark.parametrize("op", [1, 2])
@pytest.mark.parametrize("m,n,k", [(1, 4096, 4096), (2, 333, 2048), (4, 1000, 11008 - 11008 % 256), (3, 96, 512), (8, 132, 2048), (40, 256, 1024)])
def test_fused_product_equals_the_two_step_form_and_the_oracle(P, torch, fmt_name, op, m, n, k):
    fmt = oracle.FORMATS[fmt_name]
    blocks = make_weights(fmt_name, n, k, seed=7100 + n)
    x, w, eps = _inputs(op, m, k, 7200 + m)
    wts = P.Weights.upload(fmt, blocks, n, k)
    xd = torch.from_numpy(x).cuda()
    wd = torch.from_numpy(w).cuda() if w is not None else None
    fused = torch.full((m, n), float("nan"), dtype=torch.float32, device="cuda")
    P.gemm_quant_nt_pre_dev(wts, op, xd, fused, m, pre_w_dev=wd, eps=eps, mode=P.MODE_INT8)
    act = _dev_pre(P, torch, op, x, w, eps, k)
    two_step = torch.full((m, n), float("nan"), dtype=torch.float32, device="cuda")
    P.gemm_quant_nt_dev(wts, act, two_step, m, mode=P.MODE_INT8)
    P.synchronize()
    got = fused.cpu().numpy()
    assert np.array_equal(got.view(np.uint32), two_step.cpu().numpy().view(np.uint32))
    # the integer product of the oracle over the activations the device produced
    assert_close(got, oracle.matmul(fmt, blocks, act.cpu().numpy()), TOL_INT8, f"{fmt_name} op {op} {m}x{n}x{k}")
    # and end to end against the oracle's own row operation: an activation one f32 ulp apart can land on the other
    # side of an int8 rounding boundary, which moves one output by one quantisation step; bounded at matrix level
    want = oracle.matmul(fmt, blocks, _oracle_pre(op, x, w, eps))
    assert float(np.max(np.abs(got - want)) / np.sqrt(np.mean(want.astype(np.float64) ** 2))) < 5e-3
    wts.free()


def test_prologue_arguments(P, torch):
    blocks = make_weights("q4_k", 64, 2048, seed=7300)
    wts = P.Weights.upload(oracle.Q4_K, blocks, 64, 2048)
    x = torch.zeros((1, 2048), dtype=torch.float32, device="cuda")
    c = torch.zeros((1, 64), dtype=torch.float32, device="cuda")
    with pytest.raises(P.Declined):
        P.gemm_quant_nt_pre_dev(wts, 1, x, c, 1)            # rms_norm_mul without its weights
    with pytest.raises(P.Declined):
        P.gemm_quant_nt_pre_dev(wts, 9, x, c, 1, pre_w_dev=x)  # not an operation
    with pytest.raises(P.Declined):
        P.act_prologue_dev(2, x, c, 1, 96)                   # k not a multiple of 256
    wts.free()
