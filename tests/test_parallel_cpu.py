"""World-size-2 gloo tests of the multi-GPU host logic on CPU tensors: the sharding and exchange
code of fucina_b200/parallel.py with the oracle standing in for the device kernels. A sharded
result must equal the unsharded oracle bit for bit (no reduction crosses ranks)."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port() -> int:
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank: int, world: int, port: int, case: str, q):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import oracle
        from fucina_b200 import parallel as par
        from parity import make_weights

        if case == "tp":
            n, k, m = 72, 512, 5   # 72/4 = 18 column groups over 2 ranks: equal shards
            blocks = make_weights("q4_k", n, k, seed=5)
            a = np.random.default_rng(6).standard_normal((m, k)).astype(np.float32)
            lo, hi = par.shard_rows(n, world, rank)
            shard = blocks[lo:hi]
            lin = par.ColumnShardedLinear(n, lambda t: torch.from_numpy(oracle.matmul(oracle.Q4_K, shard, t.numpy())))
            got = par.ColumnShardedLinear.to_row_major(lin.forward(torch.from_numpy(a))).numpy()
            want = oracle.matmul(oracle.Q4_K, blocks, a)
            q.put((rank, bool(np.array_equal(got.view(np.uint32), want.view(np.uint32)))))
        elif case == "tp_ragged":
            n, k, m = 76, 256, 3   # 19 column groups: ranks own 40 and 36 columns
            blocks = make_weights("q8_0", n, k, seed=7)
            a = np.random.default_rng(8).standard_normal((m, k)).astype(np.float32)
            lo, hi = par.shard_rows(n, world, rank)
            shard = blocks[lo:hi]
            lin = par.ColumnShardedLinear(n, lambda t: torch.from_numpy(oracle.matmul(oracle.Q8_0, shard, t.numpy())))
            got = lin.forward(torch.from_numpy(a)).numpy()
            want = oracle.matmul(oracle.Q8_0, blocks, a)
            q.put((rank, bool(np.array_equal(got.view(np.uint32), want.view(np.uint32))) and (hi - lo) == (40 if rank == 0 else 36)))
        elif case == "ep":
            hidden, ffn, E, topk, T = 256, 256, 8, 3, 7   # T tokens per rank
            gate = make_weights("q5_k", E * ffn, hidden, seed=11)
            up = make_weights("q5_k", E * ffn, hidden, seed=12)
            down = make_weights("q5_k", E * hidden, ffn, seed=13)
            rng = np.random.default_rng(20 + rank)
            x = rng.standard_normal((T, hidden)).astype(np.float32)
            logits = rng.standard_normal((T, E)).astype(np.float32)
            sel, w = oracle.router_topk(logits, topk, True)
            per = E // world
            g_loc = gate[rank * per * ffn:(rank + 1) * per * ffn]
            u_loc = up[rank * per * ffn:(rank + 1) * per * ffn]
            d_loc = down[rank * per * hidden:(rank + 1) * per * hidden]

            def ffn_rows(rows: torch.Tensor, local_expert: torch.Tensor) -> torch.Tensor:
                r = rows.numpy()
                e = local_expert.numpy().astype(np.int64).reshape(-1, 1)
                ones = np.ones((r.shape[0], 1), np.float32)
                return torch.from_numpy(oracle.moe_ffn(oracle.Q5_K, g_loc, u_loc, d_loc, r, e, ones, per, ffn))

            moe = par.ExpertParallelMoE(E, topk, ffn_rows)
            got = moe.forward(torch.from_numpy(x), torch.from_numpy(sel), torch.from_numpy(w)).numpy()
            want = oracle.moe_ffn(oracle.Q5_K, gate, up, down, x, sel, w, E, ffn)
            ok = bool(np.array_equal(got.view(np.uint32), want.view(np.uint32)))

            # fixed-size exchange: every rank computes its experts' partial sums for all tokens
            def partial(x_all: torch.Tensor, sel_all: torch.Tensor, w_all: torch.Tensor) -> torch.Tensor:
                xa, sa, wa = x_all.numpy(), sel_all.numpy(), w_all.numpy()
                acc = np.zeros_like(xa)
                for j in range(topk):   # slot order; a slot of another rank's expert adds nothing
                    mine = (sa[:, j] // per) == rank
                    if not mine.any():
                        continue
                    rows = np.ascontiguousarray(xa[mine])
                    e = (sa[mine, j] % per).astype(np.int64).reshape(-1, 1)
                    y = oracle.moe_ffn(oracle.Q5_K, g_loc, u_loc, d_loc, rows, e, np.ascontiguousarray(wa[mine, j:j + 1]), per, ffn)
                    acc[mine] += y
                return torch.from_numpy(acc)

            scale = float(np.sqrt(np.mean(want.astype(np.float64) ** 2)))
            for chunks in (1, 7):   # one exchange, and one per token (T = 7): the pipelined form's indexing
                got2 = moe.forward_gathered(torch.from_numpy(x), torch.from_numpy(sel), torch.from_numpy(w), partial, chunks=chunks).numpy()
                ok = ok and float(np.max(np.abs(got2 - want))) <= 1e-5 * scale   # only the f32 summation order differs
            # int32 ids + float32 weights travel packed in one gather
            got3 = moe.forward_gathered(torch.from_numpy(x), torch.from_numpy(sel.astype(np.int32)), torch.from_numpy(w), partial).numpy()
            ok = ok and float(np.max(np.abs(got3 - want))) <= 1e-5 * scale
            q.put((rank, ok))
    finally:
        dist.destroy_process_group()


def _run(case: str):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, case, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=60) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert sorted(results) == [(0, True), (1, True)], results


def test_shard_rows_partition():
    sys.path.insert(0, ROOT)
    from fucina_b200.parallel import shard_rows

    for n, g in ((14336, 8), (4096, 2), (76, 2), (32000, 8), (100, 8)):
        bounds = [shard_rows(n, g, r) for r in range(g)]
        assert bounds[0][0] == 0 and bounds[-1][1] == n
        assert all(b[1] == c[0] for b, c in zip(bounds, bounds[1:]))
        assert all((hi - lo) % 4 == 0 for lo, hi in bounds)
    assert shard_rows(14336, 8, 3) == (5376, 7168)  # 1792 columns per rank at 8 GPUs
    with pytest.raises(ValueError):
        shard_rows(10, 2, 0)


def test_column_sharded_linear_equals_unsharded():
    _run("tp")


def test_column_sharded_linear_ragged_shards():
    _run("tp_ragged")


def test_expert_parallel_moe_equals_unsharded():
    _run("ep")
