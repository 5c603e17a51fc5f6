"""GPU parity of the multi-GPU forms, one process per GPU (skipped with fewer than two GPUs): the
column-sharded linear and the expert-parallel MoE layer against the same layer on one GPU, through the
Python host logic over torch.distributed and through the C ABI (fq_tp_init, fq_gemm_quant_nt_tp,
fq_moe_layer_ep in its fused peer-memory form and its NCCL form).

NVLS is switched off in the children so that a rank that dies in a failing test cannot leave a multicast
binding behind; the library's own kernels use plain peer stores and loads only."""
import os
import socket
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port() -> int:
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank: int, world: int, port: int, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import torch
    import torch.distributed as dist

    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    ok = {}
    try:
        import oracle
        from fucina_b200 import parallel as par
        from fucina_b200 import provider as P
        from parity import make_weights

        P.init(rank)
        ext = torch.cuda.ExternalStream(P.stream_ptr())

        # ---- column-sharded linear: no reduction crosses ranks, so the gathered result equals one GPU's bits
        n, k, m = 256, 2048, 3
        blocks = make_weights("q4_k", n, k, seed=31)
        a = torch.from_numpy(np.random.default_rng(32).standard_normal((m, k)).astype(np.float32)).cuda()
        full = P.Weights.upload(oracle.Q4_K, blocks, n, k)
        want = torch.empty((m, n), device="cuda")
        lo, hi = par.shard_rows(n, world, rank)
        shard = P.Weights.upload(oracle.Q4_K, blocks[lo:hi], hi - lo, k)
        y_local = torch.empty((m, hi - lo), device="cuda")
        torch.cuda.synchronize()

        def gemm(t):
            P.gemm_quant_nt_dev(shard, t, y_local, m, mode=P.MODE_INT8)
            return y_local

        with torch.cuda.stream(ext):
            P.gemm_quant_nt_dev(full, a, want, m, mode=P.MODE_INT8)
            got = par.ColumnShardedLinear.to_row_major(par.ColumnShardedLinear(n, gemm).forward(a))
        P.synchronize()
        torch.cuda.synchronize()
        ok["tp"] = bool(torch.equal(got, want))

        # ---- expert-parallel MoE: both exchange forms against the unsharded layer on this GPU
        hidden, ffn, E, topk, T = 256, 256, 8, 2, 6
        fmt = oracle.Q5_K
        gate = make_weights("q5_k", E * ffn, hidden, seed=41)
        up = make_weights("q5_k", E * ffn, hidden, seed=42)
        down = make_weights("q5_k", E * hidden, ffn, seed=43)
        rng = np.random.default_rng(50)          # the same tokens on every rank; rank r owns rows [r*T, (r+1)*T)
        x_all = rng.standard_normal((world * T, hidden)).astype(np.float32)
        sel_all, w_all = oracle.router_topk(rng.standard_normal((world * T, E)).astype(np.float32), topk, True)
        wfull = [P.Weights.upload(fmt, t, r, c, E) for t, r, c in ((gate, ffn, hidden), (up, ffn, hidden), (down, hidden, ffn))]
        xd = torch.from_numpy(x_all).cuda()
        sd = torch.from_numpy(sel_all.astype(np.int32)).cuda()
        wd = torch.from_numpy(w_all).cuda()
        ref = torch.empty((world * T, hidden), device="cuda")
        per = E // world
        wloc = [P.Weights.upload(fmt, t[rank * per * r:(rank + 1) * per * r], r, c, per)
                for t, r, c in ((gate, ffn, hidden), (up, ffn, hidden), (down, hidden, ffn))]
        torch.cuda.synchronize()

        def ffn_rows(rows, local_expert):
            R = rows.shape[0]
            o = torch.empty_like(rows)
            P.moe_layer_dev(*wloc, rows.contiguous(), R, 1, local_expert.contiguous(), torch.ones((R,), device="cuda"), o)
            return o

        def partial_rows(xa, sa, wa):
            o = torch.empty_like(xa)
            P.moe_layer_ep_dev(*wloc, xa, xa.shape[0], topk, sa.contiguous(), wa.contiguous(), rank * per, o)
            return o

        mine = slice(rank * T, (rank + 1) * T)
        moe = par.ExpertParallelMoE(E, topk, ffn_rows)
        with torch.cuda.stream(ext):
            P.moe_layer_dev(*wfull, xd, world * T, topk, sd, wd, ref)
            got_a2a = moe.forward(xd[mine].contiguous(), sd[mine].contiguous(), wd[mine].contiguous())
            got_g1 = moe.forward_gathered(xd[mine].contiguous(), sd[mine].contiguous(), wd[mine].contiguous(), partial_rows)
            got_g2 = moe.forward_gathered(xd[mine].contiguous(), sd[mine].contiguous(), wd[mine].contiguous(), partial_rows, chunks=2)
        P.synchronize()
        torch.cuda.synchronize()
        want_m = ref[mine]
        scale = float(want_m.pow(2).mean().sqrt())
        ok["ep_all_to_all"] = float((got_a2a - want_m).abs().max()) <= 1e-5 * scale
        ok["ep_gathered"] = float((got_g1 - want_m).abs().max()) <= 1e-5 * scale
        ok["ep_gathered_chunked"] = float((got_g2 - want_m).abs().max()) <= 1e-5 * scale

        # ---- the same two exchanges behind the C ABI: fq_tp_init (NCCL inside the library, peer-mapped arenas),
        # fq_gemm_quant_nt_tp and fq_moe_layer_ep in its fused form (peer stores + bounded flag waits) and its
        # NCCL baseline form
        from fucina_b200._lib import load

        P.tp_init_torch(dist, arena_bytes=256 << 20)
        ok["tp_init"] = load().fq_tp_ranks() == world and load().fq_tp_rank() == rank
        ok["peer_access"] = P.tp_peer_access()
        gathered = torch.full((world, m, hi - lo), float("nan"), device="cuda")
        P.gemm_quant_nt_tp(shard, a, gathered, m, mode=P.MODE_INT8)
        P.synchronize()
        ok["tp_c_abi"] = bool(torch.equal(gathered.permute(1, 0, 2).reshape(m, n), want))
        # tensor-arm reference of this rank's tokens on one GPU: the fused form must reproduce its bits
        T2 = 150
        rng2 = np.random.default_rng(60 + rank)
        x2 = torch.from_numpy(rng2.standard_normal((T2, hidden)).astype(np.float32)).cuda()
        s2, w2 = oracle.router_topk(rng2.standard_normal((T2, E)).astype(np.float32), topk, True)
        s2d, w2d = torch.from_numpy(s2.astype(np.int32)).cuda(), torch.from_numpy(w2).cuda()
        ref2 = torch.empty((T2, hidden), device="cuda")
        load().fq_set_moe_tensor_for_test(1)
        P.moe_layer_dev(*wfull, x2, T2, topk, s2d, w2d, ref2)
        load().fq_set_moe_tensor_for_test(-1)
        P.synchronize()
        for layer in range(3):  # consecutive layers reuse the arenas: epochs order them
            out2 = torch.full((T2, hidden), float("nan"), device="cuda")
            P.moe_layer_ep(*wloc, x2, T2, topk, s2d, w2d, out2, flags=P.EP_FUSED)
            P.synchronize()
            ok[f"ep_fused_bits_layer{layer}"] = bool(torch.equal(out2, ref2))
        out3 = torch.full((T2, hidden), float("nan"), device="cuda")
        P.moe_layer_ep(*wloc, x2, T2, topk, s2d, w2d, out3, flags=P.EP_NCCL)
        P.synchronize()
        scale2 = float(ref2.pow(2).mean().sqrt())
        ok["ep_nccl_form"] = float((out3 - ref2).abs().max()) <= 1e-5 * scale2
        dist.barrier()
        P.tp_shutdown()
    except Exception as e:  # report instead of hanging the peers
        ok["error"] = repr(e)
    finally:
        q.put((rank, ok))
        dist.destroy_process_group()


def test_multi_gpu_forms_match_one_gpu():
    import torch
    import torch.multiprocessing as mp

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    try:
        results = dict(q.get(timeout=300) for _ in procs)
    finally:
        for p in procs:
            p.join(timeout=60)
            if p.is_alive():  # a rank stuck behind a failed peer: end exactly that child
                p.kill()
    for rank, ok in results.items():
        assert "error" not in ok, (rank, ok)
        assert all(ok.values()), (rank, ok)
