"""GPU parity: streaming attention forward against the f64 oracle of the reference's own GPU tests
(src/backend/cuda.zig:3484-3556: the four prefill cases and their tolerance max(2e-3 * max(|want|, |got|), 2e-3)),
plus decode shapes (one query row, thousands of keys, splits merged by the second kernel), f32 KV with stats."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def P():
    from fucina_b200 import provider

    provider.init(0)
    return provider


def attn_f64(q, k, v, kvmap, offset, scale, window, causal):
    """cuda.zig:3527-3553 restated: per (row, head) scores over the row's key range, softmax in f64."""
    q_seq, heads, d = q.shape
    kv_seq = k.shape[0]
    out = np.zeros(q.shape, np.float64)
    stats = np.zeros((heads, q_seq, 2), np.float64)
    k64, v64, q64 = k.astype(np.float64), v.astype(np.float64), q.astype(np.float64)
    for qi in range(q_seq):
        p_abs = offset + qi
        end = min(kv_seq, p_abs + 1) if causal else kv_seq
        start = p_abs + 1 - window if (causal and window > 0 and p_abs + 1 > window) else 0
        for h in range(heads):
            kvh = int(kvmap[h])
            s = (k64[start:end, kvh] @ q64[qi, h]) * scale
            m = s.max()
            p = np.exp(s - m)
            out[qi, h] = (p @ v64[start:end, kvh]) / p.sum()
            stats[h, qi] = (m, p.sum())
    return out, stats


def check(got, want):
    tol = np.maximum(2e-3 * np.maximum(np.abs(want), np.abs(got)), 2e-3)
    assert not np.isnan(got).any()
    assert np.all(np.abs(got - want) <= tol), float(np.max(np.abs(got - want)))


@pytest.mark.parametrize("q_seq,kv_seq,heads,kv_heads,d,window,causal", [
    (64, 64, 8, 4, 64, 0, True),      # plain gqa causal
    (33, 97, 4, 4, 48, 0, True),      # chunked prefill (offset 64)
    (40, 40, 8, 2, 128, 16, True),    # sliding window
    (37, 37, 6, 3, 80, 0, False),     # bidirectional
])
def test_reference_prefill_cases(P, q_seq, kv_seq, heads, kv_heads, d, window, causal):
    rng = np.random.default_rng(41)
    q = rng.standard_normal((q_seq, heads, d)).astype(np.float32)
    k = rng.standard_normal((kv_seq, kv_heads, d)).astype(np.float16)
    v = rng.standard_normal((kv_seq, kv_heads, d)).astype(np.float16)
    kvmap = [h * kv_heads // heads for h in range(heads)]
    scale = 1.0 / np.sqrt(d)
    got = P.attn_fwd(q, k, v, kvmap, kv_seq - q_seq, scale, window, causal)
    check(got, attn_f64(q, k, v, kvmap, kv_seq - q_seq, scale, window, causal)[0])


@pytest.mark.parametrize("q_seq,kv_seq,heads,kv_heads,d,window", [
    (1, 4096, 32, 8, 128, 0),       # a decode step: the key range is split over many CTAs
    (1, 5000, 8, 8, 64, 1024),      # ragged split, sliding window
    (4, 777, 16, 2, 256, 0),        # a few rows, the largest head size
    (2, 130, 4, 1, 128, 0),         # barely more than one split
    (1, 1500, 16, 2, 64, 0),        # eight heads per kv head: two passes of four over the same tiles (tensor-core form)
    (3, 300, 10, 2, 96, 64),        # five heads per kv head: a pass of four and a pass of one
])
def test_decode_shapes_and_split_merge(P, q_seq, kv_seq, heads, kv_heads, d, window):
    rng = np.random.default_rng(42)
    q = rng.standard_normal((q_seq, heads, d)).astype(np.float32)
    k = rng.standard_normal((kv_seq, kv_heads, d)).astype(np.float16)
    v = rng.standard_normal((kv_seq, kv_heads, d)).astype(np.float16)
    kvmap = [h * kv_heads // heads for h in range(heads)]
    scale = 1.0 / np.sqrt(d)
    got, stats = P.attn_fwd(q, k, v, kvmap, kv_seq - q_seq, scale, window, True, want_stats=True)
    want, want_stats = attn_f64(q, k, v, kvmap, kv_seq - q_seq, scale, window, True)
    check(got, want)
    assert np.allclose(stats[..., 0], want_stats[..., 0], rtol=1e-5, atol=1e-5)
    assert np.allclose(stats[..., 1], want_stats[..., 1], rtol=1e-4)


def test_f32_kv_with_stats_and_a_permuted_head_map(P):
    # the f32-KV forward (cuda.zig:3558-...) and a kv map that is not the uniform grouping
    rng = np.random.default_rng(43)
    q_seq, kv_seq, heads, kv_heads, d = 19, 51, 6, 3, 72
    q = rng.standard_normal((q_seq, heads, d)).astype(np.float32)
    k = rng.standard_normal((kv_seq, kv_heads, d)).astype(np.float32)
    v = rng.standard_normal((kv_seq, kv_heads, d)).astype(np.float32)
    kvmap = [2, 0, 1, 1, 0, 2]
    got, stats = P.attn_fwd(q, k, v, kvmap, kv_seq - q_seq, 0.11, 0, True, want_stats=True)
    want, want_stats = attn_f64(q, k, v, kvmap, kv_seq - q_seq, 0.11, 0, True)
    check(got, want)
    assert np.allclose(stats, want_stats, rtol=1e-4, atol=1e-5)


def test_results_do_not_depend_on_the_grid(P):
    # the same problem twice gives the same bits (fixed merge order), and rows are independent of their neighbours
    rng = np.random.default_rng(44)
    q = rng.standard_normal((3, 8, 128)).astype(np.float32)
    k = rng.standard_normal((2000, 2, 128)).astype(np.float16)
    v = rng.standard_normal((2000, 2, 128)).astype(np.float16)
    kvmap = [h // 4 for h in range(8)]
    a = P.attn_fwd(q, k, v, kvmap, 1997, 0.09)
    b = P.attn_fwd(q, k, v, kvmap, 1997, 0.09)
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))


def test_argument_rules(P):
    q = np.zeros((1, 2, 20), np.float32)
    k = np.zeros((4, 1, 20), np.float16)
    with pytest.raises(P.Declined):
        P.attn_fwd(q, k, k, [0, 0], 3, 1.0)          # d not a multiple of 8
    q = np.zeros((1, 2, 16), np.float32)
    k = np.zeros((4, 1, 16), np.float16)
    with pytest.raises(P.Declined):
        P.attn_fwd(q, k, k, [0, 1], 3, 1.0)          # map entry outside the kv heads
