"""GPU checks of the runtime rules around the kernels: the shared-memory bound of the
small-batch kernel, stream-ordered reuse of cached scratch, long group tables, and the
completion token's wait-then-copy order."""
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


@pytest.mark.parametrize("fmt_name,k,m", [("q4_k", 28672, 16), ("q8_0", 16384, 16), ("q4_k", 28672, 5), ("tq2_0", 32768, 9)])
def test_long_rows_are_served_in_smaller_row_chunks(P, torch, fmt_name, k, m):
    # pad(m) activation records of a long row exceed the 227 KiB a CTA can hold: the entry cuts
    # the batch into chunks that fit instead of failing after the first launch
    fmt = oracle.FORMATS[fmt_name]
    n = 64
    assert P.small_batch_max_rows(fmt, k) < 16
    blocks = make_weights(fmt_name, n, k, seed=41)
    w = P.Weights.upload(fmt, blocks, n, k)
    a = acts(m, k, 42)
    ad = torch.from_numpy(a).cuda()
    cd = torch.full((m, n), float("nan"), dtype=torch.float32, device="cuda")
    P.gemm_quant_nt_dev(w, ad, cd, m, mode=P.MODE_INT8)
    P.synchronize()
    assert_close(cd.cpu().numpy(), oracle.matmul(fmt, blocks, a), TOL_INT8, f"{fmt_name} k={k} m={m}")
    # and a healthy call right after reports no stale error
    P.gemm_quant_nt_dev(w, ad[:1], cd[:1], 1, mode=P.MODE_INT8)
    P.synchronize()
    w.free()


def test_library_stream_and_user_stream_share_cached_scratch_safely(P, torch):
    # Same shape on the library stream and on a caller's stream, interleaved, no host waits in
    # between: both take their activation scratch from the same size class of the cache, so the
    # second taker must be ordered after the first one's kernels.
    n, k, m = 4096, 4096, 16
    blocks = make_weights("q4_k", n, k, seed=43)
    w = P.Weights.upload(oracle.Q4_K, blocks, n, k)
    user = torch.cuda.Stream()
    rng = np.random.default_rng(44)
    a_lib = [rng.standard_normal((m, k)).astype(np.float32) for _ in range(4)]
    a_usr = [rng.standard_normal((m, k)).astype(np.float32) for _ in range(4)]
    d_lib = [torch.from_numpy(a).cuda() for a in a_lib]
    d_usr = [torch.from_numpy(a).cuda() for a in a_usr]
    c_lib = [torch.full((m, n), float("nan"), device="cuda") for _ in range(4)]
    c_usr = [torch.full((m, n), float("nan"), device="cuda") for _ in range(4)]
    torch.cuda.synchronize()
    for i in range(4):
        P.gemm_quant_nt_dev(w, d_lib[i], c_lib[i], m, mode=P.MODE_INT8)
        P.gemm_quant_nt_dev(w, d_usr[i], c_usr[i], m, mode=P.MODE_INT8, stream=user.cuda_stream)
    P.synchronize()
    user.synchronize()
    for i in range(4):
        assert_close(c_lib[i].cpu().numpy(), oracle.matmul_fast(oracle.Q4_K, blocks, a_lib[i]), TOL_INT8, f"library stream {i}")
        assert_close(c_usr[i].cpu().numpy(), oracle.matmul_fast(oracle.Q4_K, blocks, a_usr[i]), TOL_INT8, f"user stream {i}")
    w.free()


def test_user_stream_entry_does_not_block_the_host(P, torch):
    # a *_dev call on a caller's stream returns while its kernels are still queued behind a long
    # predecessor on that stream: scratch goes back to the cache with an event, not a host wait
    import time

    n, k, m = 4096, 4096, 16
    blocks = make_weights("q4_k", n, k, seed=45)
    w = P.Weights.upload(oracle.Q4_K, blocks, n, k)
    a = torch.from_numpy(acts(m, k, 46)).cuda()
    c = torch.empty((m, n), device="cuda")
    user = torch.cuda.Stream()
    P.gemm_quant_nt_dev(w, a, c, m, mode=P.MODE_INT8, stream=user.cuda_stream)  # warm the cache and the kernel attributes
    user.synchronize()
    big = torch.empty((8192, 8192), device="cuda")
    with torch.cuda.stream(user):
        for _ in range(40):  # a few tens of milliseconds of queued work
            big @ big
        t0 = time.perf_counter()
        P.gemm_quant_nt_dev(w, a, c, m, mode=P.MODE_INT8, stream=user.cuda_stream)
        dt = time.perf_counter() - t0
        done = user.query()
    user.synchronize()
    assert not done, "the predecessor finished too early for this check to mean anything"
    assert dt < 5e-3, f"the entry waited {dt * 1e3:.1f} ms on the host"
    w.free()


def test_group_table_longer_than_the_grid_y_limit(P, torch):
    # the fused layer's integer arm on a format the streaming kernel does not take (TQ2_0 stacks): the
    # table has one entry per group of <= 16 rows of an expert; with the grid's y extent capped at 7 the
    # CTAs must stride over the ~130 entries (the same walk serves tables beyond the hardware's 65535)
    hidden, out_pe, n_expert, top_k, seq = 256, 256, 8, 2, 1000
    gate = make_weights("tq2_0", n_expert * out_pe, hidden, seed=47)
    up = make_weights("tq2_0", n_expert * out_pe, hidden, seed=48)
    down = make_weights("tq2_0", n_expert * hidden, out_pe, seed=49)
    wg = P.Weights.upload(oracle.TQ2_0, gate, out_pe, hidden, n_expert)
    wu = P.Weights.upload(oracle.TQ2_0, up, out_pe, hidden, n_expert)
    wd = P.Weights.upload(oracle.TQ2_0, down, hidden, out_pe, n_expert)
    rng = np.random.default_rng(50)
    x = rng.standard_normal((seq, hidden)).astype(np.float32)
    sel = np.stack([rng.permutation(n_expert)[:top_k] for _ in range(seq)]).astype(np.int32)
    wts = rng.random((seq, top_k)).astype(np.float32)
    from fucina_b200._lib import load

    load().fq_set_moe_tensor_for_test(0)
    load().fq_set_group_grid_limit_for_test(7)
    try:
        xd, sd, wtd = torch.from_numpy(x).cuda(), torch.from_numpy(sel).cuda(), torch.from_numpy(wts).cuda()
        od = torch.full((seq, hidden), float("nan"), device="cuda")
        P.moe_layer_dev(wg, wu, wd, xd, seq, top_k, sd, wtd, od)
        P.synchronize()
    finally:
        load().fq_set_moe_tensor_for_test(-1)
        load().fq_set_group_grid_limit_for_test(0)
    want = oracle.moe_ffn(oracle.TQ2_0, gate, up, down, x, sel.astype(np.int64), wts, n_expert, out_pe)
    assert_close(od.cpu().numpy(), want, 5e-3, "integer-arm layer with a striding table walk")
    for w in (wg, wu, wd):
        w.free()


def test_work_finish_wait_then_copy(P):
    # accelerator.Work: a token that was only waited on can still be asked for its host copy
    n, k = 64, 256
    wts = make_weights("q8_0", n, k, seed=51)
    x = acts(1, k, 52)
    wk = P.gemm_quant_nt_async(oracle.Q8_0, wts, x, n, 1, k)
    wk.finish(copy_to_host=False)
    assert np.isnan(wk.out).all()
    wk.finish(copy_to_host=True)
    assert_close(wk.out, oracle.matmul(oracle.Q8_0, wts, x), TOL_INT8, "copy after wait")
    wk.finish(copy_to_host=True)  # host_ready: a no-op
    wk.destroy()
    from fucina_b200._lib import load

    load().fq_evict_resident(wts.ctypes.data)


@pytest.mark.parametrize("fmt_name,n,m", [("q4_k", 4096, 1), ("q4_k", 4096, 4), ("q5_k", 1024, 9), ("q8_0", 4096, 2), ("q4_k", 1000, 3)])
def test_shared_input_batch_of_decode_shapes_is_one_stacked_launch(P, fmt_name, n, m):
    # Q/K/V-style batch: three matrices, one decode-sized input (src/backend/cuda.zig:2441-2492). The stack runs as
    # ONE launch of the streaming kernel; c keeps the [matrix][m][n] layout of the per-matrix form.
    fmt = oracle.FORMATS[fmt_name]
    k, batch = 4096, 3
    blocks = make_weights(fmt_name, n * batch, k, seed=53)
    a = acts(m, k, 54)
    before = P.trace_counters()["launches"]
    got = P.gemm_quant_nt_shared_a_batch(fmt, blocks, a, n, batch, cacheable=False)
    after = P.trace_counters()["launches"]
    for b in range(batch):
        want = oracle.matmul_fast(fmt, blocks[b * n:(b + 1) * n], a)
        assert_close(got[b * m:(b + 1) * m], want, TOL_INT8, f"{fmt_name} matrix {b} of the stack, m={m}")
    assert after - before <= 3  # repack + (quantise) + one product, not one product per matrix
    # the asynchronous entry takes the same route (resident weights)
    wk = P.gemm_quant_nt_async(fmt, blocks, a, n, m, k, batch=batch)
    wk.finish(copy_to_host=True)
    assert np.array_equal(wk.out.view(np.uint32), got.view(np.uint32))
    wk.destroy()
    from fucina_b200._lib import load

    load().fq_evict_resident(blocks.ctypes.data)


def test_registered_host_storage_is_used_in_place(P):
    # ensureHostRegistered (src/backend/cuda.zig:1047-1082): activations and decode-sized results in registered
    # storage skip the staging copies; results are identical, and the range can be released afterwards
    n, k = 4096, 4096
    blocks = make_weights("q4_k", n, k, seed=55)
    pool = np.zeros((1 << 20,), np.float32)  # one registered allocation holding both the input and the result
    P.host_register(pool)
    P.host_register(pool)  # a covered range is accepted again
    a = pool[1000:1000 + k].reshape(1, k)
    a[:] = acts(1, k, 56)
    c = pool[300000:300000 + n].reshape(1, n)
    c[:] = np.nan
    want = oracle.matmul_fast(oracle.Q4_K, blocks, a)
    before = P.trace_counters()
    got = P.gemm_quant_nt(oracle.Q4_K, blocks, a, n, cacheable=True, out=c)
    assert got is c
    assert_close(c, want, TOL_INT8, "blocking call on registered storage")
    c[:] = np.nan  # before the submit: the result may land in registered storage any time between submit and finish
    wk = P.gemm_quant_nt_async(oracle.Q4_K, blocks, a, n, 1, k, out=c)
    wk.finish(copy_to_host=True)
    assert_close(c, want, TOL_INT8, "async call on registered storage")
    wk.destroy()
    # unregistered storage gives the same bits
    plain = P.gemm_quant_nt(oracle.Q4_K, blocks, np.array(a), n, cacheable=True)
    assert np.array_equal(plain.view(np.uint32), c.view(np.uint32))
    P.host_unregister(pool)
    with pytest.raises(P.Declined):
        P.host_unregister(pool)
    from fucina_b200._lib import load

    load().fq_evict_resident(blocks.ctypes.data)
