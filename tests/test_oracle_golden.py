"""Pins the CPU oracle to the reference's own golden vectors and known answers.

Sources (paths inside the reference project):
  src/backend/quant/encode_golden_test.zig:1010-1026  Q4_K/Q5_K encoder bytes = ggml
  src/backend/quant/encode_golden_test.zig:1104-1140  round-trip RMSE bounds
  src/backend/quant/q8_0_tests.zig:37-82              Q8_0 known answers, tie rounding
  src/backend/quant/cold_tests.zig:1527-1529          TQ2_0 dequant = ggml bit patterns
  src/backend/quant/q4_k.zig:2060-2082, q5_k.zig:1293-1315  pattern-block dot = dense dot
"""
import numpy as np
import pytest

import oracle


def f2h_bits(x):
    return int(np.array([x], dtype=np.float16).view(np.uint16)[0])


def test_q4_k_encoder_matches_ggml_golden_bytes(goldens):
    x = goldens["input_bits"].view(np.float32)
    got = oracle.quantize_rows(oracle.Q4_K, x)
    assert np.array_equal(got, goldens["q4_k_golden"])


def test_q5_k_encoder_matches_ggml_golden_bytes(goldens):
    x = goldens["input_bits"].view(np.float32)
    got = oracle.quantize_rows(oracle.Q5_K, x)
    assert np.array_equal(got, goldens["q5_k_golden"])


def test_q6_k_encoder_matches_ggml_golden_bytes(goldens):
    # encode_golden_test.zig:515 q6_k_golden: ggml quantize_row_q6_K_ref on the same eight input vectors
    x = goldens["input_bits"].view(np.float32)
    got = oracle.quantize_rows(oracle.Q6_K, x)
    assert np.array_equal(got, goldens["q6_k_golden"])


def test_q6_k_pattern_block_dot_equals_dense_dot():
    # q6_k.zig:1279-1301: fillQ6KPattern against fillQ8KPattern; dotDense(dequant w, dequant a) == dotQ6_KQ8_K exactly
    blk = np.zeros(210, np.int64)  # assembled in wide integers, narrowed to bytes below
    scales = ((np.arange(16) % 5) - 2).astype(np.int8)
    scales[0] = 1
    blk[192:208] = scales.view(np.uint8)
    blk[208:210] = np.array([f2h_bits(1.0)], np.uint16).view(np.uint8)
    for i in range(256):  # setQ6KValue (q6_k.zig:1261-1277)
        enc = ((i % 23) - 11) + 32
        chunk, local = divmod(i, 128)
        section, l = divmod(local, 32)
        qi = chunk * 64 + (32 + l if section in (1, 3) else l)
        if section < 2:
            blk[qi] = (blk[qi] & 0xF0) | (enc & 0x0F)
        else:
            blk[qi] = (blk[qi] & 0x0F) | ((enc & 0x0F) << 4)
        hi = 128 + chunk * 32 + l
        blk[hi] = (blk[hi] & ~(0x03 << (section * 2)) & 0xFF) | (((enc >> 4) & 0x03) << (section * 2))
    blk = blk.astype(np.uint8)
    a = _q8k_pattern()
    dense_w = oracle.dequantize_rows(oracle.Q6_K, blk.reshape(1, -1), 256).reshape(-1)
    assert np.array_equal(dense_w[:16], (np.arange(16) - 11).astype(np.float32))  # the first group carries scale 1
    dense_a = a[4:260].view(np.int8).astype(np.float32)
    want = np.float32(0)
    for wv, av in zip(dense_w, dense_a):
        want = np.float32(want + np.float32(wv * av))
    assert oracle.block_dot(oracle.Q6_K, blk, a) == want


def test_golden_inputs_follow_documented_generators(goldens):
    # encode_golden_test.zig:16-31 documents the 8 input vectors; spot-check the
    # ones with closed forms so a parsing slip cannot go unnoticed.
    x = goldens["input_bits"].view(np.float32)
    i = np.arange(256, dtype=np.float32)
    assert np.array_equal(x[4], np.full(256, 0.75, np.float32))
    assert np.array_equal(x[7], np.zeros(256, np.float32))
    ramp = np.float32(-1.0) + np.float32(2.0) * i / np.float32(255.0)
    assert np.array_equal(x[0], ramp.astype(np.float32))


def test_tq2_0_dequant_matches_ggml_golden_bits(goldens):
    blocks = goldens["tq2_0_bytes"]
    d = oracle.dequantize_rows(oracle.TQ2_0, blocks.reshape(1, -1), 256 * blocks.shape[0])
    assert np.array_equal(d.view(np.uint32).reshape(-1, 256), goldens["tq2_0_expected_bits"])


def _mix32(s):
    s = np.uint32(s)
    s ^= s >> np.uint32(16)
    s = np.uint32((int(s) * 0x85EBCA6B) & 0xFFFFFFFF)
    s ^= s >> np.uint32(13)
    s = np.uint32((int(s) * 0xC2B2AE35) & 0xFFFFFFFF)
    s ^= s >> np.uint32(16)
    return s


@pytest.mark.parametrize("fmt,bound", [(oracle.Q4_K, 0.055), (oracle.Q5_K, 0.030), (oracle.Q6_K, 0.016)])
def test_round_trip_rmse_bounds(fmt, bound):
    # encode_golden_test.zig:1104-1140: U[-1,1] rows from the mix32 generator
    n = 1024
    x = np.empty(n, np.float32)
    for i in range(n):
        bits = _mix32((0x1234 + i * 0x9E3779B9) & 0xFFFFFFFF)
        x[i] = np.float32(-1.0) + np.float32(2.0) * np.float32(bits) / np.float32(4294967295.0)
    blocks = oracle.quantize_rows(fmt, x.reshape(1, n))
    y = oracle.dequantize_rows(fmt, blocks, n).reshape(-1)
    rmse = float(np.sqrt(np.mean((x.astype(np.float64) - y) ** 2)))
    assert rmse < bound


def test_q8_0_known_answer():
    src = (np.arange(32) - 16).astype(np.float32)
    expected = (np.arange(32) - 16).astype(np.int8)
    src[0], expected[0] = -127, -127
    src[31], expected[31] = 127, 127
    blocks = oracle.quantize_rows(oracle.Q8_0, src.reshape(1, 32))
    assert blocks.shape == (1, 34)
    assert int(blocks[0, :2].view(np.uint16)[0]) == f2h_bits(1.0)
    assert np.array_equal(blocks[0, 2:].view(np.int8), expected)
    back = oracle.dequantize_rows(oracle.Q8_0, blocks, 32)
    assert np.array_equal(back.reshape(-1), src)


def test_q8_0_ties_round_away_from_zero():
    src = np.zeros(32, np.float32)
    src[:7] = [127, 0.5, 1.5, 2.5, -0.5, -1.5, -2.5]
    q = oracle.quantize_rows(oracle.Q8_0, src.reshape(1, 32))[0, 2:].view(np.int8)
    assert list(q[1:7]) == [1, 2, 3, -1, -2, -3]


def _q8k_pattern():
    # q8k.zig:819-827 fillQ8KPattern
    qs = ((np.arange(256) % 17) - 8).astype(np.int8)
    bsums = qs.reshape(16, 16).astype(np.int32).sum(1).astype(np.int16)
    return np.concatenate([np.array([1.0], np.float32).view(np.uint8), qs.view(np.uint8), bsums.view(np.uint8)])


def test_q4_k_pattern_block_dot_equals_dense_dot():
    # q4_k.zig:2050-2058 fillQ4KPattern
    blk = np.zeros(144, np.uint8)
    blk[0:2] = np.array([f2h_bits(1.0)], np.uint16).view(np.uint8)
    blk[2:4] = np.array([f2h_bits(1.0)], np.uint16).view(np.uint8)
    blk[4:16] = [1, 1, 1, 1, 0, 0, 0, 0, 1, 1, 1, 1]
    i = np.arange(128)
    blk[16:] = (i % 16) | (((i + 3) % 16) << 4)
    a = _q8k_pattern()
    dense_w = oracle.dequantize_rows(oracle.Q4_K, blk.reshape(1, -1), 256).reshape(-1)
    dense_a = a[4:260].view(np.int8).astype(np.float32)
    want = np.float32(0)
    for wv, av in zip(dense_w, dense_a):
        want = np.float32(want + np.float32(wv * av))
    assert oracle.block_dot(oracle.Q4_K, blk, a) == want


def test_q5_k_pattern_block_dot_equals_dense_dot():
    # q5_k.zig:1281-1291 fillQ5KPattern
    blk = np.zeros(176, np.uint8)
    blk[0:2] = np.array([f2h_bits(1.0)], np.uint16).view(np.uint8)
    blk[4:16] = [1, 2, 3, 4, 0, 0, 0, 0, 1, 2, 3, 4]
    qh = np.zeros(32, np.uint8)
    qs = np.zeros(128, np.uint8)
    for s in range(8):
        for o in range(32):
            v = (s * 7 + o) % 32
            bi = (s // 2) * 32 + o
            if s % 2 == 0:
                qs[bi] = (qs[bi] & 0xF0) | (v & 0x0F)
            else:
                qs[bi] = (qs[bi] & 0x0F) | ((v & 0x0F) << 4)
            if v & 16:
                qh[o] |= 1 << s
    blk[16:48] = qh
    blk[48:] = qs
    a = _q8k_pattern()
    dense_w = oracle.dequantize_rows(oracle.Q5_K, blk.reshape(1, -1), 256).reshape(-1)
    # decode law check: element (s, o) carries level (s*7+o)%32 times scale s-th
    dense_a = a[4:260].view(np.int8).astype(np.float32)
    want = np.float32(0)
    for wv, av in zip(dense_w, dense_a):
        want = np.float32(want + np.float32(wv * av))
    assert oracle.block_dot(oracle.Q5_K, blk, a) == want


def test_dequant_agrees_with_gguf_py():
    # independent third-party cross-check of the decode laws
    gguf = pytest.importorskip("gguf")
    from gguf import quants

    rng = np.random.default_rng(7)
    w = (rng.standard_normal((8, 1024)) * 0.02).astype(np.float32)
    for fmt, t in ((oracle.Q8_0, gguf.GGMLQuantizationType.Q8_0), (oracle.Q4_K, gguf.GGMLQuantizationType.Q4_K),
                   (oracle.Q5_K, gguf.GGMLQuantizationType.Q5_K), (oracle.TQ2_0, gguf.GGMLQuantizationType.TQ2_0)):
        blocks = oracle.quantize_rows(fmt, w)
        ours = oracle.dequantize_rows(fmt, blocks, 1024)
        theirs = quants.dequantize(blocks, t).reshape(8, 1024)
        assert np.array_equal(ours.view(np.uint32), theirs.view(np.uint32)), fmt
    # gguf-py can also encode Q8_0: bytes must agree
    theirs = quants.quantize(w, gguf.GGMLQuantizationType.Q8_0)
    assert np.array_equal(oracle.quantize_rows(oracle.Q8_0, w), theirs.reshape(8, -1))


def test_oracle_reproduces_committed_cases(oracle_cases):
    c = oracle_cases
    for name, fmt in (("q8_0", oracle.Q8_0), ("q4_k", oracle.Q4_K), ("q5_k", oracle.Q5_K), ("tq2_0", oracle.TQ2_0)):
        blocks, a = c[f"{name}_blocks"], c[f"{name}_a"]
        k = a.shape[1]
        assert np.array_equal(oracle.dequantize_rows(fmt, blocks, k).view(np.uint32), c[f"{name}_dequant"].view(np.uint32))
        assert np.array_equal(oracle.matmul(fmt, blocks, a).view(np.uint32), c[f"{name}_matmul"].view(np.uint32))


def test_simd_baseline_equals_the_scalar_oracle():
    """The timed CPU baseline (oracle/cpu_kernels.cpp) must produce the scalar oracle's bits, for every format
    with a SIMD arm, on both threading arms (columns split for m < 32, rows split beyond) and any worker count."""
    from parity import make_weights

    def same(x, y):
        return np.array_equal(x.view(np.uint32), y.view(np.uint32))

    for name in ("q4_k", "q5_k", "q6_k", "q8_0", "tq2_0", "tq2_0_folded", "q2_0"):
        fmt = oracle.FORMATS[name]
        for n, k, m in ((64, 512, 3), (333, 2304, 5), (1000, 4096, 1), (96, 768, 40)):
            w = make_weights(name, n, k, seed=n)
            a = np.random.default_rng(k).standard_normal((m, k)).astype(np.float32)
            a[0, :8] = (1e4, -1e4, 0, 127.5, -127.5, 1e-30, 3.0, -3.0)  # saturating and tie-prone values
            want = oracle.matmul(fmt, w, a)
            for t in (1, 3, 0):
                oracle.set_threads(t)
                assert same(want, oracle.matmul_fast(fmt, w, a)), (name, n, k, m, t)
    oracle.set_threads(0)
    assert oracle.threads() >= 1
    assert all(oracle.has_simd(oracle.FORMATS[f]) == bool(oracle.has_simd(oracle.Q4_K)) for f in ("q5_k", "q6_k", "q8_0", "tq2_0"))
    # a malformed TQ2_0 block may carry code 3 (+2d): the SIMD arm must follow the scalar law there too
    w = np.random.default_rng(9).integers(0, 256, size=(16, 2 * 66), dtype=np.uint8)
    w[:, 64:66] = w[:, 130:132] = np.frombuffer(np.float16(0.01).tobytes(), np.uint8)
    a = np.random.default_rng(10).standard_normal((2, 512)).astype(np.float32)
    assert same(oracle.matmul(oracle.TQ2_0, w, a), oracle.matmul_fast(oracle.TQ2_0, w, a))


def test_simd_moe_baseline_equals_the_scalar_oracle():
    from parity import make_weights

    hidden, out_pe, n_expert, top_k, seq = 512, 256, 6, 3, 7
    for name in ("q5_k", "q4_k", "q8_0"):
        fmt = oracle.FORMATS[name]
        gate = make_weights(name, n_expert * out_pe, hidden, seed=1)
        up = make_weights(name, n_expert * out_pe, hidden, seed=2)
        down = make_weights(name, n_expert * hidden, out_pe, seed=3)
        rng = np.random.default_rng(4)
        x = rng.standard_normal((seq, hidden)).astype(np.float32)
        sel, wts = oracle.router_topk(rng.standard_normal((seq, n_expert)).astype(np.float32), top_k, True)
        want = oracle.moe_ffn(fmt, gate, up, down, x, sel, wts, n_expert, out_pe)
        got = oracle.moe_ffn_fast(fmt, gate, up, down, x, sel, wts, n_expert, out_pe)
        assert np.array_equal(want.view(np.uint32), got.view(np.uint32)), name


def test_blas_form_of_oracle_b_equals_the_scalar_one():
    # tests/parity.py:oracle_b is what the full-size GPU cases use; on a small case it must be the C oracle's number
    from parity import make_weights, oracle_b, round_bf16

    for name, k in (("q4_k", 512), ("q5_k", 256), ("q8_0", 96), ("tq2_0", 512)):
        fmt = oracle.FORMATS[name]
        b = make_weights(name, 24, k, seed=5)
        a = np.random.default_rng(6).standard_normal((7, k)).astype(np.float32)
        want = oracle.matmul_dequant_f64(fmt, b, a, round_bf16=True)
        got = oracle_b(fmt, b, a, k)
        assert np.abs(got - want).max() <= 1e-12 * max(1.0, np.abs(want).max())
    x = np.array([1.0, 1.00390625, 1.01171875, -3.0e-39, 65504.0], np.float32)  # exact, tie to even, tie up, subnormal, large
    r = round_bf16(x)
    assert r[0] == 1.0 and r[1] == 1.0 and r[2] == np.float32(1.015625)


def test_gated_pairs_follow_the_reference_formulas():
    """backend/ops.zig:150-190 restated in oracle.cpp against an independent float64 evaluation of the same
    formulas (the reference holds no stored answers for these ops): one expert, identity-like routing."""
    from parity import make_weights

    hidden, out_pe = 256, 256
    gate = make_weights("q8_0", out_pe, hidden, seed=1)
    up = make_weights("q8_0", out_pe, hidden, seed=2)
    down = make_weights("q8_0", hidden, out_pe, seed=3)
    x = (np.random.default_rng(4).standard_normal((3, hidden)) * 12).astype(np.float32)
    sel = np.zeros((3, 1), np.int64)
    w = np.ones((3, 1), np.float32)
    gv = oracle.matmul(oracle.Q8_0, gate, x).astype(np.float64)
    uv = oracle.matmul(oracle.Q8_0, up, x).astype(np.float64)
    sig = lambda v: 1 / (1 + np.exp(-v))  # noqa: E731
    forms = {
        0: uv * (gv * sig(gv)),
        1: uv * (0.5 * gv * (1 + np.tanh(0.7978845608028654 * (gv + 0.044715 * gv ** 3)))),
        2: np.clip(uv, -10, 10) * (np.minimum(gv, 10) * sig(np.minimum(gv, 10))),
        3: uv * sig(gv),
        4: 25 * np.tanh(uv * 0.04) * (4 * np.tanh(gv * 0.25) * sig(gv)),
    }
    for op, g in forms.items():
        want = oracle.matmul(oracle.Q8_0, down, g.astype(np.float32))
        got = oracle.moe_ffn(oracle.Q8_0, gate, up, down, x, sel, w, 1, out_pe, gated_op=op)
        # g differs from the f32 evaluation by rounding only; the requantisation may move single int8 steps
        assert np.abs(got - want).max() <= 2e-2 * np.abs(want).max(), op
    assert np.abs(gv).max() > 10 or np.abs(uv).max() > 10  # the clamps were exercised


def test_packed_x8_arm_equals_the_scalar_oracle():
    """The reference's eight-row packs (BlockQ4_Kx8 / BlockQ5_Kx8) restated in oracle/cpu_kernels.cpp: bit-equal to
    the compact kernels, as the reference's own tests require of its packs (src/backend/quant/q4_k_tests.zig:852-896,
    q5_k_tests.zig:92-137), on every threading split; and the layout is the reference's (one block checked byte by
    byte against the packing rule of q4_k.zig:127-192)."""
    from parity import make_weights

    if not oracle.has_simd(oracle.Q4_K):
        pytest.skip("no AVX2 on this host")

    def same(x, y):
        return np.array_equal(x.view(np.uint32), y.view(np.uint32))

    for name in ("q4_k", "q5_k", "q6_k", "tq2_0"):  # Q6_K and TQ2_0: four rows per packed block (BlockQ6_Kx4, BlockTQ2_0x4)
        fmt = oracle.FORMATS[name]
        for n, k, m in ((64, 512, 1), (328, 2304, 5), (1000, 4096, 1), (96, 768, 70)):
            w = make_weights(name, n, k, seed=n + 1)
            a = np.random.default_rng(k + 1).standard_normal((m, k)).astype(np.float32)
            a[0, :8] = (1e4, -1e4, 0, 127.5, -127.5, 1e-30, 3.0, -3.0)
            want = oracle.matmul(fmt, w, a)
            pk = oracle.PackedRows.pack(fmt, w, k)
            assert pk is not None
            for t in (1, 3, 0):
                oracle.set_threads(t)
                assert same(want, pk.matmul(a)), (name, n, k, m, t)
            pk.free()
    oracle.set_threads(0)
    # no pack for other formats or for a row count that does not fill the groups
    assert oracle.PackedRows.pack(oracle.TQ2_0_FOLDED, make_weights("tq2_0_folded", 64, 256, 1), 256) is None
    assert oracle.PackedRows.pack(oracle.TQ2_0, make_weights("tq2_0", 6, 256, 1), 256) is None
    # a malformed TQ2_0 block may carry code 3 (+2d): the packed arm follows the scalar law there too
    wbad = np.random.default_rng(9).integers(0, 256, size=(16, 2 * 66), dtype=np.uint8)
    wbad[:, 64:66] = wbad[:, 130:132] = np.frombuffer(np.float16(0.01).tobytes(), np.uint8)
    abad = np.random.default_rng(10).standard_normal((2, 512)).astype(np.float32)
    pk = oracle.PackedRows.pack(oracle.TQ2_0, wbad, 512)
    assert same(oracle.matmul(oracle.TQ2_0, wbad, abad), pk.matmul(abad))
    assert oracle.PackedRows.pack(oracle.Q4_K, make_weights("q4_k", 12, 256, 1), 256) is None
    assert oracle.PackedRows.pack(oracle.Q8_0, make_weights("q8_0", 6, 256, 1), 256) is None
    # sizes of the packed blocks: 8 x (d, dmin) + 64 scales + 64 mins + payload
    pk = oracle.PackedRows.pack(oracle.Q4_K, make_weights("q4_k", 8, 256, 2), 256)
    assert pk.nbytes == 16 + 16 + 64 + 64 + 1024
    pk = oracle.PackedRows.pack(oracle.Q5_K, make_weights("q5_k", 8, 256, 2), 256)
    assert pk.nbytes == 16 + 16 + 64 + 64 + 2048


def test_packed_x8_moe_baseline_equals_the_scalar_oracle():
    from parity import make_weights

    if not oracle.has_simd(oracle.Q5_K):
        pytest.skip("no AVX2 on this host")
    hidden, out_pe, n_expert, top_k, seq = 512, 256, 6, 3, 7
    rng = np.random.default_rng(77)
    gate = make_weights("q5_k", n_expert * out_pe, hidden, 71)
    up = make_weights("q5_k", n_expert * out_pe, hidden, 72)
    down = make_weights("q5_k", n_expert * hidden, out_pe, 73)
    x = rng.standard_normal((seq, hidden)).astype(np.float32)
    sel, w = oracle.router_topk(rng.standard_normal((seq, n_expert)).astype(np.float32), top_k, True)
    want = oracle.moe_ffn(oracle.Q5_K, gate, up, down, x, sel, w, n_expert, out_pe)
    pg, pu, pd = (oracle.PackedRows.pack(oracle.Q5_K, b, kk) for b, kk in ((gate, hidden), (up, hidden), (down, out_pe)))
    got = oracle.moe_ffn_packed(pg, pu, pd, x, sel, w, n_expert, out_pe)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    # enough pairs per expert for the batched form (pairs grouped by expert, rows four at a time): the same bits,
    # with runs of 1 to 11 rows per expert and a token that names an expert twice
    seq = 13
    x = rng.standard_normal((seq, hidden)).astype(np.float32)
    sel, w = oracle.router_topk(rng.standard_normal((seq, n_expert)).astype(np.float32), top_k, True)
    sel = np.array(sel).reshape(seq, top_k)
    sel[3, 1] = sel[3, 0]
    want = oracle.moe_ffn(oracle.Q5_K, gate, up, down, x, sel, w, n_expert, out_pe)
    for t in (1, 3, 0):
        oracle.set_threads(t)
        got = oracle.moe_ffn_packed(pg, pu, pd, x, sel, w, n_expert, out_pe)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), t
    oracle.set_threads(0)


def test_packed_q8_0x4_arm_follows_its_own_law():
    """The four-row Q8_0 pack (BlockQ8_0x4) multiplies (f32(t) * d_a) * d_w per block (src/backend/quant/q8_0.zig:1591,
    :1613, :1633), a different f32 association from the compact dot: bit-equal to that law restated in numpy, and
    within f32 rounding of the compact kernels."""
    from parity import make_weights

    if not oracle.has_simd(oracle.Q8_0):
        pytest.skip("no AVX2 on this host")
    for n, k, m in ((64, 512, 1), (100, 4096, 3), (4096, 1024, 1)):
        w = make_weights("q8_0", n, k, seed=n + 2)
        a = np.random.default_rng(k + 2).standard_normal((m, k)).astype(np.float32)
        pk = oracle.PackedRows.pack(oracle.Q8_0, w, k)
        assert pk is not None and pk.nbytes == n // 4 * (k // 32) * 136
        got = pk.matmul(a)
        # the law, block by block in f32
        wb = w.reshape(n, k // 32, 34)
        dw = wb[:, :, :2].copy().view(np.float16).astype(np.float32)[..., 0]          # [n, blocks]
        wq = wb[:, :, 2:].view(np.int8).astype(np.int32)                              # [n, blocks, 32]
        ab = oracle.quantize_acts_q8_0(a).reshape(m, k // 32, 34)
        da = ab[:, :, :2].copy().view(np.float16).astype(np.float32)[..., 0]
        aq = ab[:, :, 2:].view(np.int8).astype(np.int32)
        want = np.zeros((m, n), np.float32)
        for b in range(k // 32):
            t = (aq[:, b, :] @ wq[:, b, :].T).astype(np.float32)                     # exact in f32 (|t| < 2^24)
            want = want + (t * da[:, b][:, None]) * dw[:, b][None, :]
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), (n, k, m)
        compact = oracle.matmul(oracle.Q8_0, w, a)
        assert np.max(np.abs(got - compact)) <= 1e-5 * np.max(np.abs(compact))
        pk.free()
