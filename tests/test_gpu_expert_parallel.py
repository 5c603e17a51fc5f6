"""The fused expert-parallel MoE layer (token rows stored straight into the owning GPU's panel, result rows
stored straight into the home GPU's return panel, epoch-numbered flags with bounded waits), exercised on ONE
GPU: `fq_ep_emulate_for_test` runs `world` ranks in lockstep on the library stream, each with its own arena,
expert shard, tokens and routing. Every routed pair is multiplied by the same kernels on the same bf16 operands
whichever rank serves it, and the weighted sum runs in slot order on the home rank, so the result must equal the
one-GPU tensor arm BIT FOR BIT; that arm is held to the bf16 oracle in tests/test_gpu_tensor.py.
The multi-process form (real peers over NVLink, NCCL rendezvous) is covered by tests/test_gpu_parallel.py on
two GPUs."""
import numpy as np
import pytest

import oracle
from parity import TOL_TENSOR, make_weights

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


def build_case(P, torch, fmt_name, hidden, out_pe, n_expert, top_k, world, seq, seed):
    fmt = oracle.FORMATS[fmt_name]
    gate = make_weights(fmt_name, n_expert * out_pe, hidden, seed + 1)
    up = make_weights(fmt_name, n_expert * out_pe, hidden, seed + 2)
    down = make_weights(fmt_name, n_expert * hidden, out_pe, seed + 3)
    per = n_expert // world
    full = [P.Weights.upload(fmt, gate, out_pe, hidden, n_expert), P.Weights.upload(fmt, up, out_pe, hidden, n_expert),
            P.Weights.upload(fmt, down, hidden, out_pe, n_expert)]
    shards = []
    for r in range(world):
        shards.append([P.Weights.upload(fmt, gate[r * per * out_pe:(r + 1) * per * out_pe], out_pe, hidden, per),
                       P.Weights.upload(fmt, up[r * per * out_pe:(r + 1) * per * out_pe], out_pe, hidden, per),
                       P.Weights.upload(fmt, down[r * per * hidden:(r + 1) * per * hidden], hidden, out_pe, per)])
    rng = np.random.default_rng(seed)
    xs, sels, wts = [], [], []
    for r in range(world):
        x = rng.standard_normal((seq, hidden)).astype(np.float32)
        sel, w = oracle.router_topk(rng.standard_normal((seq, n_expert)).astype(np.float32), top_k, True)
        xs.append(x), sels.append(sel.astype(np.int32)), wts.append(w)
    return (gate, up, down), full, shards, xs, sels, wts


def single_gpu_tensor_arm(P, torch, full, x, sel, w, top_k):
    from fucina_b200._lib import load

    seq, hidden = x.shape
    out = torch.full((seq, hidden), float("nan"), device="cuda")
    load().fq_set_moe_tensor_for_test(1)
    try:
        P.moe_layer_dev(*full, torch.from_numpy(x).cuda(), seq, top_k, torch.from_numpy(sel).cuda(), torch.from_numpy(w).cuda(), out)
        P.synchronize()
    finally:
        load().fq_set_moe_tensor_for_test(-1)
    return out.cpu().numpy()


@pytest.mark.parametrize("fmt_name,hidden,out_pe,n_expert,top_k,world,seq", [
    ("q5_k", 512, 256, 16, 4, 2, 96),
    ("q5_k", 512, 256, 16, 4, 8, 40),     # two experts per rank, ragged runs
    ("q4_k", 256, 512, 8, 2, 4, 130),     # expert runs longer than one 128-token tile
    ("q8_0", 256, 256, 4, 2, 4, 33),      # one expert per rank
    ("q6_k", 512, 256, 8, 2, 4, 70),      # the six-bit K-quant (the down tensors of mixed K-quant files)
    ("q5_k", 2048, 768, 128, 8, 8, 64),   # the benchmark layer: 16 experts per rank
    ("q5_k", 512, 256, 8, 3, 1, 50),      # a single rank: every panel is its own
])
def test_emulated_ranks_equal_the_one_gpu_tensor_arm(P, torch, fmt_name, hidden, out_pe, n_expert, top_k, world, seq):
    host, full, shards, xs, sels, wts = build_case(P, torch, fmt_name, hidden, out_pe, n_expert, top_k, world, seq, seed=600)
    xd = [torch.from_numpy(x).cuda() for x in xs]
    sd = [torch.from_numpy(s).cuda() for s in sels]
    wd = [torch.from_numpy(w).cuda() for w in wts]
    od = [torch.full((seq, hidden), float("nan"), device="cuda") for _ in range(world)]
    torch.cuda.synchronize()
    arena = 64 * 1024 + seq * top_k * hidden * 4 + world * seq * top_k * (hidden * 2 + 8) + (1 << 20)
    # two layers back to back over the same arenas: the second finds the first one's rows, flags and tables in place
    P.ep_emulate_for_test([s[0] for s in shards], [s[1] for s in shards], [s[2] for s in shards], xd, seq, top_k, sd, wd, od, arena, layers=2)
    fmt = oracle.FORMATS[fmt_name]
    gate, up, down = host
    for r in range(world):
        got = od[r].cpu().numpy()
        want = single_gpu_tensor_arm(P, torch, full, xs[r], sels[r], wts[r], top_k)
        assert np.isfinite(got).all()
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), f"rank {r} of {world} differs from the one-GPU tensor arm"
    # and against the CPU oracle of the tensor arm on one rank's tokens (bound relative to the output scale)
    r = world - 1
    ref = oracle.moe_ffn_bf16(fmt, gate, up, down, xs[r], sels[r].astype(np.int64), wts[r], n_expert, out_pe)
    rms = float(np.sqrt(np.mean(ref.astype(np.float64) ** 2)))
    assert float(np.max(np.abs(od[r].cpu().numpy() - ref))) / rms <= TOL_TENSOR
    for w in full + [w for s in shards for w in s]:
        w.free()


def test_skewed_routing_every_token_to_one_rank(P, torch):
    # all pairs land on rank 1's experts: the other panels stay empty, rank 1 receives world * seq * top_k rows
    fmt_name, hidden, out_pe, n_expert, top_k, world, seq = "q5_k", 256, 256, 8, 2, 4, 24
    host, full, shards, xs, sels, wts = build_case(P, torch, fmt_name, hidden, out_pe, n_expert, top_k, world, seq, seed=610)
    per = n_expert // world
    for s in sels:
        s[:, 0], s[:, 1] = per, per + 1
    xd = [torch.from_numpy(x).cuda() for x in xs]
    sd = [torch.from_numpy(s).cuda() for s in sels]
    wd = [torch.from_numpy(w).cuda() for w in wts]
    od = [torch.full((seq, hidden), float("nan"), device="cuda") for _ in range(world)]
    arena = 64 * 1024 + seq * top_k * hidden * 4 + world * seq * top_k * (hidden * 2 + 8) + (1 << 20)
    P.ep_emulate_for_test([s[0] for s in shards], [s[1] for s in shards], [s[2] for s in shards], xd, seq, top_k, sd, wd, od, arena)
    for r in range(world):
        want = single_gpu_tensor_arm(P, torch, full, xs[r], sels[r], wts[r], top_k)
        assert np.array_equal(od[r].cpu().numpy().view(np.uint32), want.view(np.uint32))
    # an arena that cannot hold that many rows: every rank reaches the same verdict from the same count table, nothing
    # is written past a panel, and the layer ends with the capacity status
    ret_bytes = (seq * top_k * hidden * 4 + 255) & ~255
    small = 64 * 1024 + ret_bytes + 512 + 140 * (hidden * 2 + 8)  # room for 128 of the 192 rows rank 1 would receive
    with pytest.raises(P.DeviceError) as e:
        P.ep_emulate_for_test([s[0] for s in shards], [s[1] for s in shards], [s[2] for s in shards], xd, seq, top_k, sd, wd, od, small)
    assert e.value.code == -3
    # the context stays usable
    P.ep_emulate_for_test([s[0] for s in shards], [s[1] for s in shards], [s[2] for s in shards], xd, seq, top_k, sd, wd, od, arena)
    for w in full + [w for s in shards for w in s]:
        w.free()


def test_entries_decline_before_tp_init(P, torch):
    n, k = 64, 256
    w = P.Weights.upload(oracle.Q4_K, make_weights("q4_k", n, k, 1), n, k)
    a = torch.zeros((1, k), device="cuda")
    c = torch.zeros((1, n), device="cuda")
    from fucina_b200._lib import load

    if load().fq_tp_ranks() == 0:
        with pytest.raises(P.Declined):
            P.gemm_quant_nt_tp(w, a, c, 1)
        assert load().fq_tp_rank() == -1 and load().fq_tp_peer_access() == 0
    w.free()


def test_a_rank_that_never_publishes_ends_in_a_timeout_status_not_a_hang(P, torch):
    # failure detection without a fault: the last rank's count row is dropped, so no flag ever arrives for it; every
    # rank's wait is bounded (about a second), gives up, records the time-out status, and the remaining kernels of
    # the layer fall through. The context stays usable.
    import time

    fmt_name, hidden, out_pe, n_expert, top_k, world, seq = "q5_k", 256, 256, 4, 2, 2, 16
    host, full, shards, xs, sels, wts = build_case(P, torch, fmt_name, hidden, out_pe, n_expert, top_k, world, seq, seed=620)
    xd = [torch.from_numpy(x).cuda() for x in xs]
    sd = [torch.from_numpy(s).cuda() for s in sels]
    wd = [torch.from_numpy(w).cuda() for w in wts]
    od = [torch.full((seq, hidden), 5.0, device="cuda") for _ in range(world)]
    arena = 64 * 1024 + seq * top_k * hidden * 4 + world * seq * top_k * (hidden * 2 + 8) + (1 << 20)
    args = ([s[0] for s in shards], [s[1] for s in shards], [s[2] for s in shards], xd, seq, top_k, sd, wd, od, arena)
    t0 = time.perf_counter()
    with pytest.raises(P.DeviceError) as e:
        P.ep_emulate_for_test(*args, layers=-1)
    assert e.value.code == -2  # FQ_ERR_TIMEOUT
    assert time.perf_counter() - t0 < 30.0
    assert all(float(o.min()) == 5.0 and float(o.max()) == 5.0 for o in od)  # no output was produced from a partial exchange
    P.ep_emulate_for_test(*args)  # and the next layer runs normally
    want = single_gpu_tensor_arm(P, torch, full, xs[0], sels[0], wts[0], top_k)
    assert np.array_equal(od[0].cpu().numpy().view(np.uint32), want.view(np.uint32))
    for w in full + [w for s in shards for w in s]:
        w.free()
