"""GPU parity, part 3: the provider surface with HOST buffers -- residency,
async completion tokens, the grouped MoE entry, the fused MoE layer and the
router -- mirroring the reference's own provider tests
(src/backend/cuda.zig:3057-3462, :3639; src/llm/gemma/moe_tests.zig:40-204)."""
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


def acts(m, k, seed):
    return np.random.default_rng(seed).standard_normal((m, k)).astype(np.float32)


@pytest.mark.parametrize("fmt_name", ["q8_0", "q4_k", "q5_k", "tq2_0"])
def test_blocking_gemm_transient_rhs(P, fmt_name):
    fmt = oracle.FORMATS[fmt_name]
    n, k, m = 68, 512, 4
    blocks = make_weights(fmt_name, n, k, seed=1)
    a = acts(m, k, 2)
    got = P.gemm_quant_nt(fmt, blocks, a, n, cacheable=False)
    assert_close(got, oracle.matmul(fmt, blocks, a), TOL_INT8, fmt_name)


def test_resident_rhs_crosses_pcie_once(P):
    n, k = 96, 1024
    blocks = make_weights("q4_k", n, k, seed=3)
    a = acts(1, k, 4)
    before = P.trace_counters()
    y1 = P.gemm_quant_nt(oracle.Q4_K, blocks, a, n, cacheable=True)
    mid = P.trace_counters()
    y2 = P.gemm_quant_nt(oracle.Q4_K, blocks, a, n, cacheable=True)
    after = P.trace_counters()
    assert mid["resident_adopts"] == before["resident_adopts"] + 1
    assert after["resident_hits"] == mid["resident_hits"] + 1
    # second call moved only the activation row and the result
    assert after["h2d_bytes"] - mid["h2d_bytes"] == k * 4
    assert after["d2h_bytes"] - mid["d2h_bytes"] == n * 4
    assert np.array_equal(y1, y2)
    assert_close(y1, oracle.matmul(oracle.Q4_K, blocks, a), TOL_INT8, "resident")
    # an interior row range of the adopted bytes resolves to the same device copy
    sub = blocks[32:64]
    y3 = P.gemm_quant_nt(oracle.Q4_K, sub, a, 32, cacheable=True)
    assert np.array_equal(y3, y1[:, 32:64])
    assert P.trace_counters()["resident_adopts"] == mid["resident_adopts"]
    from fucina_b200._lib import load

    assert load().fq_evict_resident(blocks.ctypes.data) == 0


def test_alloc_resident_round_trip(P):
    import ctypes as C

    from fucina_b200._lib import load

    lib = load()
    n, k = 64, 512
    blocks = make_weights("q5_k", n, k, seed=5)
    p = lib.fq_alloc_resident(blocks.size)
    assert p
    C.memmove(p, blocks.ctypes.data, blocks.size)
    view = np.ctypeslib.as_array(C.cast(p, C.POINTER(C.c_uint8)), shape=(blocks.size,))
    a = acts(2, k, 6)
    got = P.gemm_quant_nt(oracle.Q5_K, view, a, n, cacheable=True)
    assert_close(got, oracle.matmul(oracle.Q5_K, blocks, a), TOL_INT8, "owned resident")
    assert lib.fq_resident_bytes() > 0
    lib.fq_free_resident(p)


def test_vram_budget_refusal(P):
    # mirrors src/backend/cuda.zig:3639: over budget -> decline, nothing written
    from fucina_b200._lib import load

    lib = load()
    n, k = 64, 512
    blocks = make_weights("q4_k", n, k, seed=7)
    a = acts(1, k, 8)
    lib.fq_set_vram_budget(16)
    try:
        out = np.full((1, n), 123.0, np.float32)
        with pytest.raises(P.Declined) as e:
            P.gemm_quant_nt(oracle.Q4_K, blocks, a, n, cacheable=True, out=out)
        assert e.value.code == 3
        assert (out == 123.0).all()
        assert lib.fq_alloc_resident(1 << 20) is None
    finally:
        lib.fq_set_vram_budget(1 << 40)
    got = P.gemm_quant_nt(oracle.Q4_K, blocks, a, n, cacheable=True)
    assert_close(got, oracle.matmul(oracle.Q4_K, blocks, a), TOL_INT8, "after budget restore")
    lib.fq_evict_resident(blocks.ctypes.data)


def test_shared_input_batch(P):
    # src/backend/cuda.zig:3243-3247: m=65, n=68, batch=2
    n, k, m, batch = 68, 512, 65, 2
    blocks = make_weights("q4_k", n * batch, k, seed=9)
    a = acts(m, k, 10)
    got = P.gemm_quant_nt_shared_a_batch(oracle.Q4_K, blocks, a, n, batch, cacheable=False)
    for b in range(batch):
        # 65 rows is past the decode kernels' batch: the automatic mode multiplies on the tensor cores,
        # whose oracle is the f64 product of bf16-rounded operands (the reference's own check at this
        # shape compares with an f64 dequantised product at 1e-2, src/backend/cuda.zig:3016-3044)
        want = oracle.matmul_dequant_f64(oracle.Q4_K, blocks[b * n:(b + 1) * n], a, round_bf16=True)
        assert_close(got[b * m:(b + 1) * m], want, 1e-2, f"batch {b}")


def test_async_dependency_chain_without_host_read(P):
    # src/backend/cuda.zig:3346-3462: y = W2 . (W1 . x) with the intermediate never read by the host
    n1, k1, n2 = 512, 256, 68
    w1 = make_weights("q8_0", n1, k1, seed=11)
    w2 = make_weights("q4_k", n2, n1, seed=12)
    x = acts(1, k1, 13)
    work1 = P.gemm_quant_nt_async(oracle.Q8_0, w1, x, n1, 1, k1)
    work2 = P.gemm_quant_nt_async(oracle.Q4_K, w2, None, n2, 1, n1, dep=work1)
    assert work1.device_ptr() != 0
    work2.finish(copy_to_host=True)
    work1.finish(copy_to_host=False)
    h = oracle.matmul(oracle.Q8_0, w1, x)
    want = oracle.matmul(oracle.Q4_K, w2, h)
    # the device intermediate differs from the oracle's by f32 ulps, which the second
    # activation quantisation can amplify to one int8 step on a few elements
    assert_close(work2.out, want, 2e-2, "chained")
    assert np.isnan(work1.out).all()  # discarded without a copy
    work2.destroy()
    work1.destroy()
    from fucina_b200._lib import load

    load().fq_evict_resident(w1.ctypes.data)
    load().fq_evict_resident(w2.ctypes.data)


def _page_aligned(shape):
    """float32 array on a 4096-byte boundary spanning whole pages (what host registration wants)."""
    count = int(np.prod(shape))
    raw = np.zeros(((count * 4 + 4095) // 4096 + 1) * 4096, np.uint8)
    off = (-raw.ctypes.data) % 4096
    return raw[off:off + count * 4].view(np.float32).reshape(shape)


def test_async_chain_through_registered_storage(P):
    # the producer's result is copied into its caller's registered storage right behind the product, and the
    # consumer chained on it still reads the device copy: the intermediate row never travels back up
    n1, k1, n2 = 512, 256, 68
    w1 = make_weights("q8_0", n1, k1, seed=21)
    w2 = make_weights("q4_k", n2, n1, seed=22)
    x = acts(1, k1, 23)
    h_out = _page_aligned((1, n1))
    h_out[:] = np.nan
    P.host_register(h_out)
    try:
        P.gemm_quant_nt(oracle.Q8_0, w1, x, n1, cacheable=True)  # adopt both weight matrices first
        P.gemm_quant_nt(oracle.Q4_K, w2, acts(1, n1, 24), n2, cacheable=True)
        before = P.trace_counters()
        work1 = P.gemm_quant_nt_async(oracle.Q8_0, w1, x, n1, 1, k1, out=h_out)
        work2 = P.gemm_quant_nt_async(oracle.Q4_K, w2, None, n2, 1, n1, dep=work1)
        work2.finish(copy_to_host=True)
        work1.finish(copy_to_host=True)
        h = oracle.matmul(oracle.Q8_0, w1, x)
        assert_close(h_out, h, TOL_INT8, "producer, into registered storage")
        assert_close(work2.out, oracle.matmul(oracle.Q4_K, w2, h), 2e-2, "chained through registered storage")
        # only the first product's activations went up; both results came down
        after = P.trace_counters()
        assert after["h2d_bytes"] - before["h2d_bytes"] == k1 * 4
        assert after["d2h_bytes"] - before["d2h_bytes"] == (n1 + n2) * 4
        work2.destroy()
        work1.destroy()
    finally:
        P.synchronize()
        P.host_unregister(h_out)
    from fucina_b200._lib import load

    load().fq_evict_resident(w1.ctypes.data)
    load().fq_evict_resident(w2.ctypes.data)


@pytest.mark.parametrize("registered", [False, True])
def test_prepared_async_calls_overlap_and_repeat(P, registered):
    # four products of different sizes queued back to back, finished afterwards, over several steps with changing
    # activations: uploads run on their own stream behind the compute stream's products, results land in `out`
    # (through page-locked staging, or, with registered storage, copied into it directly)
    shapes = [(256, 512), (1024, 512), (68, 512), (4096, 512)]
    ws = [make_weights("q4_k", n, k, seed=40 + i) for i, (n, k) in enumerate(shapes)]
    xs = [_page_aligned((1, k)) for n, k in shapes]
    outs = [_page_aligned((1, n)) for n, k in shapes]
    for i, x in enumerate(xs):
        x[:] = acts(1, x.shape[1], 50 + i)
    if registered:
        for arr in xs + outs:
            P.host_register(arr)
    calls = [P.PreparedGemmAsync(oracle.Q4_K, w, x, n, 1, k, out=o) for w, x, o, (n, k) in zip(ws, xs, outs, shapes)]
    for step in range(3):
        for x in xs:
            x *= np.float32(1.0 + 0.5 * step)  # same storage, new values every step
        for c in calls:
            c.out[:] = np.nan
            c.submit()
        with pytest.raises(RuntimeError):
            calls[0].submit()  # one product in flight per prepared call
        for c, w, x in zip(calls, ws, xs):
            assert_close(c.finish(), oracle.matmul(oracle.Q4_K, w, x), TOL_INT8, f"prepared async step {step}")
    with pytest.raises(RuntimeError):
        calls[0].finish()
    if registered:
        P.synchronize()
        for arr in xs + outs:
            P.host_unregister(arr)
    from fucina_b200._lib import load

    for w in ws:
        load().fq_evict_resident(w.ctypes.data)


def test_async_slots_decline_when_exhausted(P):
    n, k = 64, 256
    w = make_weights("q8_0", n, k, seed=14)
    x = acts(1, k, 15)
    works = []
    try:
        for _ in range(8):
            works.append(P.gemm_quant_nt_async(oracle.Q8_0, w, x, n, 1, k))
        with pytest.raises(P.Declined) as e:
            P.gemm_quant_nt_async(oracle.Q8_0, w, x, n, 1, k)
        assert e.value.code == 5
    finally:
        for wk in works:
            wk.finish()
            wk.destroy()
    from fucina_b200._lib import load

    load().fq_evict_resident(w.ctypes.data)


def _grouped_case(P, fmt_name, n_out, k, ms, mode, seed=16):
    """Run `gemmQGroupedNt` over per-expert row counts `ms` cut into the reference's 32-row tiles
    (src/llm/gemma/moe.zig:773-787) and return (blocks, a, got)."""
    fmt = oracle.FORMATS[fmt_name]
    blocks = make_weights(fmt_name, n_out * len(ms), k, seed=seed)
    rows = sum(ms)
    a = acts(rows, k, seed + 1)
    from fucina_b200._lib import load

    lib = load()
    lib.fq_set_grouped_tensor_for_test(mode)
    lib.fq_qmoe_lock()
    try:
        pin, pout = P.qmoe_stage(rows * k, rows * n_out)
        pin[:] = a.reshape(-1)
        pout[:] = np.nan
        tiles, base = [], 0
        for e, m in enumerate(ms):
            for t in range((m + 31) // 32):  # {expert, group base, group rows, tile index}: llm/gemma/moe.zig:773-787
                tiles.append((e, base, m, t))
            base += m
        P.gemm_q_grouped_nt(fmt, blocks, n_out, k, tiles)
        got = np.array(pout).reshape(rows, n_out)
    finally:
        lib.fq_qmoe_unlock()
        lib.fq_set_grouped_tensor_for_test(-1)
    return blocks, a, got


@pytest.mark.parametrize("mode", [-1, 0, 1])
@pytest.mark.parametrize("fmt_name", ["q4_k", "q5_k", "q8_0"])
def test_grouped_tiles(P, fmt_name, mode):
    # src/backend/cuda.zig:3157-3185: 4 experts, n=64, k=2B, per-expert m = {1,7,33,40}. By run length (-1) the runs
    # of 33 and 40 rows multiply on the tensor cores and the runs of 1 and 7 rows on the integer kernel; the seam
    # pins either arm for all runs.
    fmt = oracle.FORMATS[fmt_name]
    n_out, k = 64, 512
    ms = [1, 7, 33, 40]
    blocks, a, got = _grouped_case(P, fmt_name, n_out, k, ms, mode)
    base = 0
    for e, m in enumerate(ms):
        w = blocks[e * n_out:(e + 1) * n_out]
        tensor = mode == 1 or (mode == -1 and m >= 17)
        if tensor:  # bf16 operands: the reference's own bound for its grouped kernel (src/backend/cuda.zig:3016-3044)
            assert_close(got[base:base + m], oracle.matmul_dequant_f64(fmt, w, a[base:base + m], round_bf16=True), 1e-2, f"{fmt_name} expert {e} (tensor)")
        else:
            assert_close(got[base:base + m], oracle.matmul(fmt, w, a[base:base + m]), TOL_INT8, f"{fmt_name} expert {e} (int8)")
        base += m


@pytest.mark.parametrize("mode", [0, 1])
def test_grouped_long_runs_are_merged_from_32_row_tiles(P, mode):
    # four experts of 300 rows each arrive as ten tiles per expert; the tiles of an expert merge into one run
    n_out, k = 256, 1024
    ms = [300, 300, 300, 300]
    before = P.trace_counters()["launches"]
    blocks, a, got = _grouped_case(P, "q4_k", n_out, k, ms, mode, seed=18)
    launches = P.trace_counters()["launches"] - before
    base = 0
    for e, m in enumerate(ms):
        w = blocks[e * n_out:(e + 1) * n_out]
        if mode:
            assert_close(got[base:base + m], oracle.matmul_dequant_f64(oracle.Q4_K, w, a[base:base + m], round_bf16=True), 1e-2, f"expert {e}")
        else:
            assert_close(got[base:base + m], oracle.matmul_fast(oracle.Q4_K, w, a[base:base + m]), TOL_INT8, f"expert {e}")
        base += m
    assert launches <= 4  # repack, then one conversion or quantisation pass and one product: not a launch per tile


@pytest.mark.parametrize("tile", [(0, 0, 40, 2), (0, 0, 0, 0), (0, -1, 8, 0), (-1, 0, 8, 0), (0, 0, 8, -1)])
def test_grouped_malformed_tiles_decline(P, tile):
    # a tile index at or beyond the group's rows (32 * tile_m >= m), empty groups and negative fields are refused
    # before anything is launched: the output panel keeps its contents
    n_out, k = 64, 512
    blocks = make_weights("q4_k", n_out, k, seed=19)
    from fucina_b200._lib import load

    lib = load()
    lib.fq_qmoe_lock()
    try:
        pin, pout = P.qmoe_stage(64 * k, 64 * n_out)
        pin[:] = 0.0
        pout[:] = 7.0
        with pytest.raises(P.Declined):
            P.gemm_q_grouped_nt(oracle.Q4_K, blocks, n_out, k, [(0, 0, 8, 0), tile])
        assert (np.array(pout) == 7.0).all()
    finally:
        lib.fq_qmoe_unlock()


def _moe_case(fmt_name, hidden, out_pe, n_expert, top_k, seq, seed):
    rng = np.random.default_rng(seed)
    gate = make_weights(fmt_name, n_expert * out_pe, hidden, seed + 1)
    up = make_weights(fmt_name, n_expert * out_pe, hidden, seed + 2)
    down = make_weights(fmt_name, n_expert * hidden, out_pe, seed + 3)
    x = rng.standard_normal((seq, hidden)).astype(np.float32)
    logits = rng.standard_normal((seq, n_expert)).astype(np.float32)
    sel, w = oracle.router_topk(logits, top_k, True)
    return gate, up, down, x, logits, sel, w


@pytest.mark.parametrize("fmt_name,hidden,out_pe,n_expert,top_k,seq", [
    ("q5_k", 256, 256, 4, 2, 37),     # src/llm/gemma/moe_tests.zig:56-62 scaled to whole blocks
    ("q5_k", 512, 768, 16, 4, 1),     # decode
    ("q5_k", 512, 768, 16, 4, 40),    # experts with more rows than one pass
    ("q4_k", 256, 512, 8, 2, 9),
    ("q4_k", 2048, 768, 8, 4, 12),    # Qwen3-MoE expert shape: runs of 3-8 rows take the tensor-core block product
    ("q5_k", 2048, 768, 32, 8, 2),    # two tokens, K split across the warps of an item
    ("q8_0", 256, 128, 8, 3, 5),
])
def test_moe_layer_matches_oracle(P, fmt_name, hidden, out_pe, n_expert, top_k, seq):
    fmt = oracle.FORMATS[fmt_name]
    gate, up, down, x, _, sel, w = _moe_case(fmt_name, hidden, out_pe, n_expert, top_k, seq, seed=50)
    wg = P.Weights.upload(fmt, gate, out_pe, hidden, n_expert)
    wu = P.Weights.upload(fmt, up, out_pe, hidden, n_expert)
    wd = P.Weights.upload(fmt, down, hidden, out_pe, n_expert)
    from fucina_b200._lib import load

    load().fq_set_moe_tensor_for_test(0)   # the int8 arm is the one this oracle restates; larger batches would pick tensor cores
    try:
        got = P.moe_layer(wg, wu, wd, x, sel, w)
    finally:
        load().fq_set_moe_tensor_for_test(-1)
    want = oracle.moe_ffn(fmt, gate, up, down, x, sel, w, n_expert, out_pe)
    # expf on the device and in the oracle may differ by an ulp, and the requantisation
    # of g can turn that into one int8 step on isolated elements: the layer bound is the
    # f32 one with that step allowed for
    assert_close(got, want, 5e-3, f"moe {fmt_name} seq={seq}")
    for h in (wg, wu, wd):
        h.free()


@pytest.mark.parametrize("tensor_arm,seq", [(0, 5), (0, 40), (1, 300)])
def test_moe_expert_shards_sum_to_the_layer(P, torch, tensor_arm, seq):
    """Two expert shards on one device: each serves half the experts, skips the other half's
    pairs, and the partial outputs add up to the unsharded layer (f32 summation order aside)."""
    from fucina_b200._lib import load

    hidden, out_pe, n_expert, top_k = 256, 512, 8, 3
    fmt = oracle.Q5_K
    gate, up, down, x, _, sel, w = _moe_case("q5_k", hidden, out_pe, n_expert, top_k, seq, seed=80)
    sel[0, :] = (0, 1, 2)          # a token served by shard 0 alone: shard 1 must write zeros for it
    xd = torch.from_numpy(x).cuda()
    sd = torch.from_numpy(sel.astype(np.int32)).cuda()
    wd_ = torch.from_numpy(w).cuda()
    load().fq_set_moe_tensor_for_test(tensor_arm)
    try:
        full = P.Weights.upload(fmt, gate, out_pe, hidden, n_expert), P.Weights.upload(fmt, up, out_pe, hidden, n_expert), \
            P.Weights.upload(fmt, down, hidden, out_pe, n_expert)
        want = torch.full((seq, hidden), float("nan"), device="cuda")
        P.moe_layer_dev(*full, xd, seq, top_k, sd, wd_, want)
        total = torch.zeros((seq, hidden), device="cuda")
        per = n_expert // 2
        for r in range(2):
            sl_gu = slice(r * per * out_pe, (r + 1) * per * out_pe)
            sl_d = slice(r * per * hidden, (r + 1) * per * hidden)
            shard = P.Weights.upload(fmt, gate[sl_gu], out_pe, hidden, per), P.Weights.upload(fmt, up[sl_gu], out_pe, hidden, per), \
                P.Weights.upload(fmt, down[sl_d], hidden, out_pe, per)
            part = torch.full((seq, hidden), float("nan"), device="cuda")
            P.moe_layer_ep_dev(*shard, xd, seq, top_k, sd, wd_, r * per, part)
            P.synchronize()
            if r == 1:
                assert float(part[0].abs().max()) == 0.0
            total += part
            for h in shard:
                h.free()
        P.synchronize()
        got, ref = total.cpu().numpy(), want.cpu().numpy()
        assert np.isfinite(got).all()
        scale = float(np.sqrt(np.mean(ref.astype(np.float64) ** 2)))
        assert float(np.max(np.abs(got - ref))) <= 1e-5 * scale
        for h in full:
            h.free()
    finally:
        load().fq_set_moe_tensor_for_test(-1)


def test_moe_output_need_not_be_16_byte_aligned(P, torch):
    """The combine writes four columns per thread when the output rows are 16-byte aligned and one
    column per thread otherwise; both give the same bits."""
    hidden, out_pe, n_expert, top_k, seq = 256, 256, 4, 2, 9
    gate, up, down, x, _, sel, w = _moe_case("q4_k", hidden, out_pe, n_expert, top_k, seq, seed=90)
    ws = [P.Weights.upload(oracle.Q4_K, b, n, k, n_expert) for b, n, k in ((gate, out_pe, hidden), (up, out_pe, hidden), (down, hidden, out_pe))]
    xd = torch.from_numpy(x).cuda()
    sd = torch.from_numpy(sel.astype(np.int32)).cuda()
    wd_ = torch.from_numpy(w).cuda()
    aligned = torch.full((seq * hidden,), float("nan"), device="cuda")
    backing = torch.full((seq * hidden + 4,), float("nan"), device="cuda")
    shifted = backing[1:1 + seq * hidden]          # 4 bytes past a 16-byte boundary
    assert aligned.data_ptr() % 16 == 0 and shifted.data_ptr() % 16 == 4
    P.moe_layer_dev(*ws, xd, seq, top_k, sd, wd_, aligned)
    P.moe_layer_dev(*ws, xd, seq, top_k, sd, wd_, shifted)
    P.synchronize()
    a, b = aligned.cpu().numpy(), shifted.cpu().numpy()
    assert np.isfinite(a).all() and np.array_equal(a.view(np.uint32), b.view(np.uint32))
    assert np.isnan(backing[0].item()) and np.isnan(backing[-1].item())  # nothing written outside the rows
    for h in ws:
        h.free()


def test_moe_token_may_name_an_expert_twice(P):
    """A routing row that repeats an expert makes that expert's run longer than the batch; the
    row-group table must split it rather than drop rows."""
    from fucina_b200._lib import load

    gate, up, down, x, _, sel, w = _moe_case("q5_k", 256, 256, 4, 2, 2, seed=61)
    sel[0, :] = (1, 1)
    sel[1, :] = (0, 1)
    wg = P.Weights.upload(oracle.Q5_K, gate, 256, 256, 4)
    wu = P.Weights.upload(oracle.Q5_K, up, 256, 256, 4)
    wd = P.Weights.upload(oracle.Q5_K, down, 256, 256, 4)
    load().fq_set_moe_tensor_for_test(0)
    try:
        got = P.moe_layer(wg, wu, wd, x, sel, w)
    finally:
        load().fq_set_moe_tensor_for_test(-1)
    want = oracle.moe_ffn(oracle.Q5_K, gate, up, down, x, sel, w, 4, 256)
    assert_close(got, want, 5e-3, "repeated expert")
    for h in (wg, wu, wd):
        h.free()


def test_moe_rejects_bad_expert_index(P):
    gate, up, down, x, _, sel, w = _moe_case("q5_k", 256, 256, 4, 2, 3, seed=60)
    wg = P.Weights.upload(oracle.Q5_K, gate, 256, 256, 4)
    wu = P.Weights.upload(oracle.Q5_K, up, 256, 256, 4)
    wd = P.Weights.upload(oracle.Q5_K, down, 256, 256, 4)
    bad = sel.copy()
    bad[1, 0] = 4
    with pytest.raises(P.Declined):
        P.moe_layer(wg, wu, wd, x, bad, w)


def test_router_topk_matches_oracle(P, torch):
    rng = np.random.default_rng(70)
    logits = rng.standard_normal((33, 128)).astype(np.float32)
    logits[0, 5] = logits[0, 9] = logits[0].max() + 1.0   # exact tie: the earlier index wins
    logits[1, :] = 0.25                                   # all equal: first k indices
    for normalize in (True, False):
        sel, w = oracle.router_topk(logits, 8, normalize)
        ld = torch.from_numpy(logits).cuda()
        sd = torch.zeros((33, 8), dtype=torch.int32, device="cuda")
        wd = torch.zeros((33, 8), dtype=torch.float32, device="cuda")
        P.router_topk_dev(ld, 33, 128, 8, normalize, sd, wd)
        P.synchronize()
        assert np.array_equal(sd.cpu().numpy(), sel.astype(np.int32))
        np.testing.assert_allclose(wd.cpu().numpy(), w, rtol=2e-6, atol=0)
    assert list(sel[1]) == list(range(8))
    assert sel[0, 0] == 5 and sel[0, 1] == 9


def test_bounded_device_wait_reports_timeout_and_context_survives(P):
    """Failure detection without a fault: a device-side wait that can never succeed gives up after its
    limit, the host reads FQ_ERR_TIMEOUT (-2) at the next synchronisation, and later work runs normally."""
    from fucina_b200._lib import load

    lib = load()
    P.synchronize()                              # nothing pending from earlier tests
    assert lib.fq_selftest_bounded_wait(0) == 1  # declined: limit out of range
    assert lib.fq_selftest_bounded_wait(20000) == 0
    assert lib.fq_synchronize() == -2            # the wait ran out and said so
    assert lib.fq_synchronize() == 0             # reported once, then cleared
    n, k = 64, 512
    blocks = make_weights("q4_k", n, k, seed=90)
    a = acts(2, k, 91)
    got = P.gemm_quant_nt(oracle.Q4_K, blocks, a, n, cacheable=False)
    assert_close(got, oracle.matmul(oracle.Q4_K, blocks, a), TOL_INT8, "after a reported time-out")


@pytest.mark.parametrize("tensor_arm,seq", [(0, 9), (1, 150)])
@pytest.mark.parametrize("gated_op", [1, 2, 3, 4])
def test_moe_gated_ops_fused_gate_up_and_a_q8_0_down(P, gated_op, tensor_arm, seq):
    """Gemma's expert FFN as the reference's GPU arm sees it (src/llm/gemma/moe.zig:696-901): ONE fused gate_up tensor
    [E][2 * out_pe][hidden] in Q4_K (gate rows first), GeGLU, and a Q8_0 down tensor; plus the other gated ops of
    backend/ops.zig:89-107. The two halves of the fused tensor are row views of the uploaded stack."""
    from fucina_b200._lib import load

    hidden, out_pe, n_expert, top_k = 256, 256, 4, 2
    gate = make_weights("q4_k", n_expert * out_pe, hidden, seed=71)
    up = make_weights("q4_k", n_expert * out_pe, hidden, seed=72)
    down = make_weights("q8_0", n_expert * hidden, out_pe, seed=73)
    rb = gate.shape[1]
    fused = np.concatenate([gate.reshape(n_expert, out_pe, rb), up.reshape(n_expert, out_pe, rb)], axis=1).reshape(n_expert * 2 * out_pe, rb)
    w_fused = P.Weights.upload(oracle.Q4_K, fused, 2 * out_pe, hidden, n_expert)
    wg, wu = w_fused.view(0, out_pe), w_fused.view(out_pe, out_pe)
    wd = P.Weights.upload(oracle.Q8_0, down, hidden, out_pe, n_expert)
    rng = np.random.default_rng(74)
    x = (rng.standard_normal((seq, hidden)) * 12).astype(np.float32)  # wide enough for the +-10 clamps to bite
    sel, w = oracle.router_topk(rng.standard_normal((seq, n_expert)).astype(np.float32), top_k, True)
    load().fq_set_moe_tensor_for_test(tensor_arm)
    try:
        got = P.moe_layer(wg, wu, wd, x, sel, w, gated_op=gated_op)
    finally:
        load().fq_set_moe_tensor_for_test(-1)
    if tensor_arm:
        want = oracle.moe_ffn_bf16(oracle.Q4_K, gate, up, down, x, sel, w, n_expert, out_pe, gated_op=gated_op, fmt_down=oracle.Q8_0)
        rms = float(np.sqrt(np.mean(want.astype(np.float64) ** 2)))
        assert np.isfinite(got).all() and float(np.max(np.abs(got - want))) / rms <= 1e-2
    else:
        want = oracle.moe_ffn(oracle.Q4_K, gate, up, down, x, sel, w, n_expert, out_pe, gated_op=gated_op, fmt_down=oracle.Q8_0)
        assert_close(got, want, 5e-3, f"gated op {gated_op}, integer arm")
    for h in (wg, wu, wd, w_fused):
        h.free()


def test_moe_rejects_unknown_gated_op_and_mismatched_pair(P):
    gate, up, down, x, _, sel, w = _moe_case("q5_k", 256, 256, 4, 2, 3, seed=62)
    wg = P.Weights.upload(oracle.Q5_K, gate, 256, 256, 4)
    wu4 = P.Weights.upload(oracle.Q4_K, make_weights("q4_k", 4 * 256, 256, 63), 256, 256, 4)
    wd = P.Weights.upload(oracle.Q5_K, down, 256, 256, 4)
    with pytest.raises(P.Declined):
        P.moe_layer(wg, wg, wd, x, sel, w, gated_op=9)
    with pytest.raises(P.Declined):
        P.moe_layer(wg, wu4, wd, x, sel, w)  # gate and up must share a format
    for h in (wg, wu4, wd):
        h.free()


@pytest.mark.parametrize("planes,seq", [(1, 5), (2, 1), (2, 37), (3, 20)])
def test_moe_layer_over_ptqtp_expert_stacks(P, torch, planes, seq):
    """`MoePtqtpRhs` (src/exec/moe.zig:51-78): every projection of an expert is K ternary planes; each product is the
    plane dots added per element in plane order (`moePtqtpTileDotRange`, :591-631)."""
    hidden, out_pe, n_expert, top_k = 512, 256, 6, 2
    rng = np.random.default_rng(90 + planes)

    def stack(rows, k, p):
        trits = rng.integers(-1, 2, size=(n_expert * rows, k)).astype(np.int8)
        scales = np.abs(rng.standard_normal((n_expert * rows, k // 256)) * 0.02 / (3 ** p)).astype(np.float32)
        return oracle.pack_ptqtp_plane(trits, scales)

    gate = [stack(out_pe, hidden, p) for p in range(planes)]
    up = [stack(out_pe, hidden, p) for p in range(planes)]
    down = [stack(hidden, out_pe, p) for p in range(planes)]
    x = rng.standard_normal((seq, hidden)).astype(np.float32)
    sel, w = oracle.router_topk(rng.standard_normal((seq, n_expert)).astype(np.float32), top_k, True)
    wg = [P.Weights.upload(oracle.TQ2_0, b, out_pe, hidden, n_expert) for b in gate]
    wu = [P.Weights.upload(oracle.TQ2_0, b, out_pe, hidden, n_expert) for b in up]
    wd = [P.Weights.upload(oracle.TQ2_0, b, hidden, out_pe, n_expert) for b in down]
    out = torch.full((seq, hidden), float("nan"), device="cuda")
    P.moe_layer_ptqtp_dev(wg, wu, wd, torch.from_numpy(x).cuda(), seq, top_k, torch.from_numpy(sel.astype(np.int32)).cuda(),
                          torch.from_numpy(w).cuda(), out)
    P.synchronize()
    want = oracle.moe_ffn_ptqtp(gate, up, down, x, sel, w, n_expert, out_pe)
    assert_close(out.cpu().numpy(), want, 5e-3, f"PTQTP experts, {planes} plane(s), seq {seq}")
    if planes == 1:  # one plane is the plain TQ2_0 expert layer
        assert np.array_equal(want, oracle.moe_ffn(oracle.TQ2_0, gate[0], up[0], down[0], x, sel, w, n_expert, out_pe))
    for h in wg + wu + wd:
        h.free()
