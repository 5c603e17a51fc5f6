"""Benchmark of the quantized-matmul hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (N = 1): the Q4_K decode GEMV stack the headline metric is quoted on
-- Llama-7B-style projections at batch 1, K = 4096 -> N in {4096, 11008, 4096,
32000}. One step = the four products once. Weights are seeded N(0, 0.02) f32
rows pushed through the library's own device-side Q4_K encoder (byte-identical
to the reference encoder, see tests/test_gpu_formats.py); activations are
seeded N(0, 1). A pool of distinct weight copies larger than 4x the L2 is
rotated so every step streams its weights from HBM.

`value`   GB/s of algorithmic bytes (GGUF weight bytes + activations + outputs)
          with everything resident in HBM, CUDA-event timed on the library
          stream.
`e2e`     the same metric through the blocking C-ABI call with HOST buffers
          (resident weights; activations go up and results come down every
          call), wall-clock timed between device synchronisations.
`roofline` achieved bytes/s of the dominant kernel alone (the 32000 x 4096
          product), CUDA events around back-to-back graph replays over the
          rotated weight copies, against the measured HBM copy bandwidth.
`cpu_baseline` the CPU restatement of the reference kernels on the host cores.

With --gpus N > 1 every rank serves its own decode stream from its own weight
replica (weak scaling, no collective on the data path); time is the max over
ranks.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

K = 4096
STACK_N = [4096, 11008, 4096, 32000]
Q4_K = 2
ROW_BYTES = K // 256 * 144
L2_BYTES = 126 * 1024 * 1024


def stack_bytes(batch: int = 1) -> int:
    """Algorithmic bytes of one step: weights once, activations in, outputs out."""
    return sum(n * ROW_BYTES + batch * K * 4 + batch * n * 4 for n in STACK_N)


def measured_peaks() -> tuple[float, str]:
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except Exception:
                self.proc.kill()

    def summary(self) -> dict:
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            if len(r) < 9:
                continue
            try:
                sm.append(float(r[1]))
                mx.append(float(r[2]))
            except ValueError:
                continue
            for name, v in zip(names, r[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def dist_setup(n_gpus: int):
    """torch.distributed over NCCL when launched under torchrun; plain single process otherwise."""
    import torch

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        import torch.distributed as dist

        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    return rank, world, local


def barrier(world: int):
    import torch

    if world > 1:
        import torch.distributed as dist

        dist.barrier()
    torch.cuda.synchronize()


def max_over_ranks(x: float, world: int) -> float:
    if world == 1:
        return x
    import torch
    import torch.distributed as dist

    t = torch.tensor([x], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


class Stack:
    """One copy of the decode stack: device weights, and host bytes for the host-buffer arm."""

    def __init__(self, P, torch, seed: int, keep_host: bool):
        self.weights, self.host = [], []
        for i, n in enumerate(STACK_N):
            g = torch.Generator(device="cuda").manual_seed(1000 + 100 * 1 + 10 * seed + i)
            w = torch.randn((n, K), generator=g, device="cuda", dtype=torch.float32) * 0.02
            blocks = torch.empty(n * ROW_BYTES, dtype=torch.uint8, device="cuda")
            torch.cuda.synchronize()  # torch's stream made w; the encoder runs on the library stream
            P.quantize_rows_dev(Q4_K, w, n, K, blocks)  # the library's device-side Q4_K encoder
            P.synchronize()
            self.weights.append(P.Weights.from_device(Q4_K, blocks, n, K))
            if keep_host:
                self.host.append(blocks.cpu().numpy().reshape(n, ROW_BYTES))
            del w, blocks


def run_ours(args) -> dict:
    import torch

    from fucina_b200 import provider as P

    rank, world, local = dist_setup(args.gpus)
    P.init(local)
    ext = torch.cuda.ExternalStream(P.stream_ptr())
    batch = max(1, min(16, getattr(args, "batch", 1)))  # 1 is the headline; 4 and 16 are the other decode batches of the config
    n_copies = max(2, -(-4 * L2_BYTES // sum(n * ROW_BYTES for n in STACK_N)))  # pool >= 4x L2
    stacks = [Stack(P, torch, s, keep_host=True) for s in range(n_copies)]
    g = torch.Generator(device="cuda").manual_seed(2000 + 100 * 1 + rank)
    xs = [torch.randn((batch, K), generator=g, device="cuda", dtype=torch.float32) for _ in STACK_N]
    ys = [torch.empty((batch, n), device="cuda", dtype=torch.float32) for n in STACK_N]
    torch.cuda.synchronize()

    def step_dev(i: int):
        st = stacks[i % n_copies]
        for w, x, y in zip(st.weights, xs, ys):
            P.gemm_quant_nt_dev(w, x, y, batch, mode=P.MODE_INT8)

    for i in range(args.warmup):
        step_dev(i)
    P.synchronize()

    # One CUDA graph per weight copy: a step is four microsecond-scale kernels, so the
    # eager launch cost of a Python caller would otherwise be what gets timed.
    # A decode loop replays one graph per token holding hundreds of such kernels; here one "cycle"
    # graph holds a step over each weight copy in turn (n_copies steps), so consecutive kernels keep
    # their programmatic-launch overlap across step boundaries as they would inside a model's graph.
    # Single-step graphs serve the remainder when the step count is not a multiple of n_copies.
    step_graphs = []
    for c in range(n_copies):
        with P.capture() as cap:
            step_dev(c)
        step_graphs.append(cap.graph)
    with P.capture() as cap:
        for c in range(n_copies):
            step_dev(c)
    step_cycle = cap.graph
    # the dominant kernel alone (the 32000 x 4096 lm_head product), one launch per copy
    big = max(range(len(STACK_N)), key=lambda i: STACK_N[i])
    big_graphs = []
    for c in range(n_copies):
        with P.capture() as cap:
            P.gemm_quant_nt_dev(stacks[c].weights[big], xs[big], ys[big], batch, mode=P.MODE_INT8)
        big_graphs.append(cap.graph)
    with P.capture() as cap:
        for c in range(n_copies):
            P.gemm_quant_nt_dev(stacks[c].weights[big], xs[big], ys[big], batch, mode=P.MODE_INT8)
    big_cycle = cap.graph

    def timed_graphs(cycle, graphs, steps: int) -> float:
        """Exactly `steps` steps: whole cycles of n_copies steps, then single-step graphs."""
        barrier(world)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(ext):
            e0.record()
            for _ in range(steps // n_copies):
                cycle.launch()
            for i in range(steps % n_copies):
                graphs[i].launch()
            e1.record()
        P.synchronize()
        barrier(world)
        return max_over_ranks(e0.elapsed_time(e1), world)

    for i in range(max(args.warmup, 3)):
        step_graphs[i % n_copies].launch()
        big_graphs[i % n_copies].launch()
        step_cycle.launch()
        big_cycle.launch()
    P.synchronize()

    # ---- value: resident inputs, CUDA events on the library stream ----
    with ClockSampler(local) as clk:
        ms = timed_graphs(step_cycle, step_graphs, args.steps)
        # keep the sampler busy for short runs so it sees the clocks under load
        t_end = time.time() + 0.6
        while time.time() < t_end:
            step_cycle.launch()
            P.synchronize()
    # one decode kernel per product with the activation quantisation fused in (batch <= 4); wider batches
    # quantise in a kernel of their own first
    launches = args.steps * len(STACK_N) * (1 if batch <= 4 else 2)
    bytes_step = stack_bytes(batch)
    value = world * bytes_step * args.steps / (ms * 1e-3) / 1e9

    # ---- roofline: the dominant kernel alone, back-to-back launches over the rotated copies ----
    k_n = args.steps
    k_ms = timed_graphs(big_cycle, big_graphs, k_n)
    peak, peak_src = measured_peaks()
    per_launch_bytes = STACK_N[big] * ROW_BYTES + batch * K * 4 + batch * STACK_N[big] * 4
    achieved = per_launch_bytes / (k_ms / k_n * 1e-3) / 1e9
    roofline = {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak, "unit": "GB/s",
                "frac": round(achieved / peak, 4),
                # dram__bytes_read + dram__bytes_write of one profiler capture of the same kernel on a 65536-row
                # matrix (151.31 MB + 3.46 MB), scaled to this launch by rows (traffic is proportional to rows)
                "traffic": int((151_309_056 + 3_462_656) * STACK_N[big] / 65536),
                "traffic_source": "ncu capture of a 65536 x 4096 case, scaled by rows",
                "kernel": "decode_rows_kernel<Q4_K, MB=1, fused act-quant> on 32000x4096",
                "peak_source": peak_src, "launches_timed": k_n,
                "timing": "CUDA events around back-to-back launches (graph replay, consecutive launches overlap by programmatic dependent launch)", "us_per_launch": round(k_ms / k_n * 1e3, 3),
                "bytes_per_launch": per_launch_bytes, "frac_of_8TBs": round(achieved / 8000.0, 4)}

    # ---- e2e: blocking C-ABI call, host buffers, resident weights ----
    host_x = [x.cpu().numpy() for x in xs]
    host_y = [np.empty((batch, n), np.float32) for n in STACK_N]

    def step_host(i: int):
        st = stacks[i % n_copies]
        for hw, x, y, n in zip(st.host, host_x, host_y, STACK_N):
            P.gemm_quant_nt(Q4_K, hw, x, n, cacheable=True, out=y)

    for i in range(max(args.warmup, n_copies)):  # first touch adopts each copy's weights
        step_host(i)
    barrier(world)
    t0 = time.perf_counter()
    for i in range(args.steps):
        step_host(i)
    P.synchronize()
    e2e_s = max_over_ranks(time.perf_counter() - t0, world)
    barrier(world)
    e2e = {"value": round(world * bytes_step * args.steps / e2e_s / 1e9, 2), "unit": "GB/s",
           "h2d_bytes_per_step": len(STACK_N) * batch * K * 4, "d2h_bytes_per_step": sum(STACK_N) * batch * 4,
           "ms_per_step": round(e2e_s / args.steps * 1e3, 4), "timing": "wall clock between device syncs",
           "call": "fq_gemm_quant_nt (blocking), one call per product"}

    # the same step through the asynchronous entry (the reference's gemmQuantNtAsync + Work.finish): the
    # four products of a step are submitted back to back and finished afterwards, so uploads, kernels and
    # downloads of different products overlap
    def step_host_async(i: int):
        st = stacks[i % n_copies]
        works = [P.gemm_quant_nt_async(Q4_K, hw, x, n, batch, K, out=y) for hw, x, y, n in zip(st.host, host_x, host_y, STACK_N)]
        for wk in works:
            wk.finish(copy_to_host=True)
            wk.destroy()

    for i in range(max(args.warmup, n_copies)):
        step_host_async(i)
    barrier(world)
    t0 = time.perf_counter()
    for i in range(args.steps):
        step_host_async(i)
    P.synchronize()
    async_s = max_over_ranks(time.perf_counter() - t0, world)
    barrier(world)
    e2e["async_submit"] = {"value": round(world * bytes_step * args.steps / async_s / 1e9, 2), "unit": "GB/s",
                           "ms_per_step": round(async_s / args.steps * 1e3, 4),
                           "call": "fq_gemm_quant_nt_async x4, then fq_work_finish x4"}

    out = {
        "metric": "quant GEMV HBM GB/s", "value": round(value, 1), "unit": "GB/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(ms / args.steps, 5), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "int8xq4 -> f32", "data": "synthetic",
        "config": {"workload": f"Q4_K decode GEMV stack, batch {batch}, K=4096 -> N in {{4096,11008,4096,32000}}",
                   "bytes_per_step": bytes_step, "weight_copies_rotated": n_copies,
                   "l2_policy": f"inputs larger than L2: {n_copies} distinct weight copies ({n_copies * bytes_step >> 20} MiB) rotated",
                   "parallelism": f"dp{world} replicas" if world > 1 else "single GPU"},
        "frac_of_8TBs": round(value / world / 8000.0, 4),
        "roofline": roofline, "e2e": e2e, "gpu_launches": launches, "clocks": clk.summary(),
    }
    if rank == 0 and world == 1 and not args.no_cpu:
        out["cpu_baseline"] = cpu_baseline(stacks[0].host, host_x, budget_s=10.0)
    return out if rank == 0 else {}


def cpu_baseline(host_w, host_x, budget_s: float) -> dict:
    """The CPU restatement of the reference kernels (activations to Q8_K, dotQ4_KQ8_K rows,
    output columns split over the host threads) on one stack copy, a few passes."""
    import oracle

    cores = os.cpu_count() or 1
    bytes_step = stack_bytes(1)
    oracle.matmul_fast(Q4_K, host_w[0][:256], host_x[0])  # load the library
    t0 = time.perf_counter()
    passes = 0
    while True:
        for w, x in zip(host_w, host_x):
            oracle.matmul_fast(Q4_K, w, x)
        passes += 1
        dt = time.perf_counter() - t0
        if dt > budget_s or passes >= 5000:
            break
    return {"value": round(bytes_step * passes / dt / 1e9, 3), "unit": "GB/s", "cores": cores, "kind": "port",
            "sample": f"{passes} pass(es) of the full stack (4 products, batch 1), {dt:.1f} s, "
                      + ("AVX2 block dots" if oracle.has_simd(Q4_K) else "scalar block dots"),
            "ms_per_step": round(dt / passes * 1e3, 2)}


def run_reference(args) -> dict:
    """The reference's CPU path for the same workload: its Zig kernels cannot be built here
    (no Zig toolchain), so the timed code is their C++ restatement in oracle/."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return {}
    import oracle

    rng = np.random.default_rng(1100)
    # seeded N(0,0.02) weights through the restated reference encoder; a bounded row sample
    # of each matrix keeps a step short (all host threads are used)
    frac = 8
    ws = [oracle.quantize_rows(Q4_K, (rng.standard_normal((n // frac, K)) * 0.02).astype(np.float32)) for n in STACK_N]
    xs = [rng.standard_normal((1, K)).astype(np.float32) for _ in STACK_N]
    bytes_step = sum(w.shape[0] * ROW_BYTES + K * 4 + w.shape[0] * 4 for w in ws)

    def step():
        for w, x in zip(ws, xs):
            oracle.matmul_fast(Q4_K, w, x)

    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = time.perf_counter() - t0
    value = round(bytes_step * args.steps / dt / 1e9, 3)
    cores = os.cpu_count() or 1
    sample = (f"rows/{frac} of each stack matrix per step, {args.steps} steps, {dt:.1f} s, "
              + ("AVX2 block dots" if oracle.has_simd(Q4_K) else "scalar block dots"))
    return {
        "impl": "reference", "metric": "quant GEMV HBM GB/s", "value": value, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(dt / args.steps * 1e3, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8xq4 -> f32", "data": "synthetic",
        "config": {"workload": "Q4_K decode GEMV stack, batch 1, K=4096 -> N in {4096,11008,4096,32000}",
                   "bytes_per_step": bytes_step, "note": "CPU restatement of the reference kernels; Zig toolchain absent"},
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }


def run_profile_case(args) -> dict:
    """A small case of the same decode kernel for profiler captures: one Q4_K matrix
    larger than the L2 (65536 x 4096, 151 MB), a handful of launches, no CPU leg."""
    import torch

    from fucina_b200 import provider as P

    P.init(0)
    n = 65536
    g = torch.Generator(device="cuda").manual_seed(77)
    w = torch.randn((n, K), generator=g, device="cuda", dtype=torch.float32) * 0.02
    blocks = torch.empty(n * ROW_BYTES, dtype=torch.uint8, device="cuda")
    torch.cuda.synchronize()
    P.quantize_rows_dev(Q4_K, w, n, K, blocks)
    P.synchronize()
    wt = P.Weights.from_device(Q4_K, blocks, n, K)
    x = torch.randn((1, K), generator=g, device="cuda", dtype=torch.float32)
    y = torch.empty((1, n), device="cuda", dtype=torch.float32)
    torch.cuda.synchronize()
    for _ in range(args.warmup):
        P.gemm_quant_nt_dev(wt, x, y, 1, mode=P.MODE_INT8)
    P.synchronize()
    P.kernel_timing(True)
    for _ in range(args.steps):
        P.gemm_quant_nt_dev(wt, x, y, 1, mode=P.MODE_INT8)
    P.synchronize()
    ms, cnt = P.kernel_times()
    nbytes = n * ROW_BYTES + K * 4 + n * 4
    return {"workload": "profile case: Q4_K GEMV 65536x4096 batch 1", "launches": cnt, "bytes_per_launch": nbytes,
            "avg_kernel_us": round(ms / max(cnt, 1) * 1e3, 2), "GBps": round(nbytes / (ms / max(cnt, 1) * 1e-3) / 1e9, 1)}


def run_profile_q8(args) -> dict:
    """The Q8_0 decode kernel for profiler captures: one 32000 x 4096 matrix (139 MB, larger than
    the L2), payload staged by 128-byte-swizzled tensor copies, a handful of launches."""
    import torch

    from fucina_b200 import formats as F
    from fucina_b200 import provider as P

    P.init(0)
    n = 32000
    w = _dev_weights(P, torch, F.Q8_0, n, K, 1100)
    g = torch.Generator(device="cuda").manual_seed(78)
    x = torch.randn((1, K), generator=g, device="cuda", dtype=torch.float32)
    y = torch.empty((1, n), device="cuda", dtype=torch.float32)
    torch.cuda.synchronize()
    for _ in range(args.warmup):
        P.gemm_quant_nt_dev(w, x, y, 1, mode=P.MODE_INT8)
    P.synchronize()
    P.kernel_timing(True)
    for _ in range(args.steps):
        P.gemm_quant_nt_dev(w, x, y, 1, mode=P.MODE_INT8)
    P.synchronize()
    ms, cnt = P.kernel_times()
    nbytes = n * (K // 32 * 34) + K * 4 + n * 4
    return {"workload": "profile case: Q8_0 GEMV 32000x4096 batch 1", "launches": cnt, "bytes_per_launch": nbytes,
            "avg_kernel_us": round(ms / max(cnt, 1) * 1e3, 2), "GBps": round(nbytes / (ms / max(cnt, 1) * 1e-3) / 1e9, 1)}


def run_profile_moe(args) -> dict:
    """One prefill-sized expert layer for profiler launch lists: Q5_K, hidden 2048, ffn 768, 128 experts, top-8,
    1024 tokens (8192 routed rows), plain launches (no graph), router outside the timed loop."""
    import torch

    from fucina_b200 import formats as F
    from fucina_b200 import provider as P

    P.init(0)
    hidden, ffn, n_expert, top_k, seq = 2048, 768, 128, 8, 1024
    gate = _dev_weights(P, torch, F.Q5_K, ffn, hidden, 1300, n_expert)
    up = _dev_weights(P, torch, F.Q5_K, ffn, hidden, 1301, n_expert)
    down = _dev_weights(P, torch, F.Q5_K, hidden, ffn, 1302, n_expert)
    g = torch.Generator(device="cuda").manual_seed(5)
    x = torch.randn((seq, hidden), generator=g, device="cuda")
    logits = torch.randn((seq, n_expert), generator=g, device="cuda")
    sel = torch.empty((seq, top_k), dtype=torch.int32, device="cuda")
    w = torch.empty((seq, top_k), device="cuda")
    out = torch.empty((seq, hidden), device="cuda")
    torch.cuda.synchronize()
    P.router_topk_dev(logits, seq, n_expert, top_k, True, sel, w)
    P.synchronize()

    def layer():
        P.moe_layer_dev(gate, up, down, x, seq, top_k, sel, w, out)

    ms = _timed(P, torch, layer, args.steps, args.warmup)
    return {"workload": "profile case: Q5_K MoE layer 2048/768, 128 experts, top-8, 1024 tokens (plain launches)", "ms": round(ms, 4),
            "tok_per_s": round(seq / ms * 1e3, 1)}


def _timed(P, torch, fn, steps: int, warmup: int) -> float:
    """milliseconds per call of fn() on the library stream (CUDA events)."""
    ext = torch.cuda.ExternalStream(P.stream_ptr())
    for _ in range(warmup):
        fn()
    P.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(ext):
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
    P.synchronize()
    return e0.elapsed_time(e1) / steps


def _dev_weights(P, torch, fmt: int, n: int, k: int, seed: int, n_mats: int = 1):
    from fucina_b200 import formats as F

    g = torch.Generator(device="cuda").manual_seed(seed)
    rb = F.row_bytes(fmt, k)
    blocks = torch.empty(n_mats * n * rb, dtype=torch.uint8, device="cuda")
    for e in range(n_mats):  # one matrix at a time keeps the f32 staging small
        w = torch.randn((n, k), generator=g, device="cuda", dtype=torch.float32) * 0.02
        torch.cuda.synchronize()
        P.quantize_rows_dev(fmt, w, n, k, blocks[e * n * rb:(e + 1) * n * rb])
        P.synchronize()
    return P.Weights.from_device(fmt, blocks, n, k, n_mats)


def run_extra(args) -> list[dict]:
    """The other configurations of the hot path, one JSON line each (information; the
    driver's headline run is the default workload)."""
    import torch

    from fucina_b200 import formats as F
    from fucina_b200 import provider as P

    P.init(0)
    peak_hbm, _ = measured_peaks()
    out = []
    g = torch.Generator(device="cuda").manual_seed(5)
    if args.workload in ("q8_0", "all"):
        n = k = 4096
        copies = [_dev_weights(P, torch, F.Q8_0, n, k, 1000 + i) for i in range(30)]  # 535 MB > 4x L2
        x = torch.randn((1, k), generator=g, device="cuda")
        y = torch.empty((1, n), device="cuda")
        torch.cuda.synchronize()
        with P.capture() as cap:
            for w in copies:
                P.gemm_quant_nt_dev(w, x, y, 1, mode=P.MODE_INT8)
        ms = _timed(P, torch, cap.graph.launch, max(args.steps // 10, 5), 3) / len(copies)
        nbytes = n * (k // 32 * 34) + 4 * k + 4 * n
        out.append({"workload": "Q8_0 GEMV 4096x4096 batch 1 (30 rotated copies)", "us_per_launch": round(ms * 1e3, 3),
                    "GBps": round(nbytes / ms / 1e6, 1), "frac_of_measured_hbm": round(nbytes / ms / 1e6 / peak_hbm, 4)})
        del copies, cap
        # the lm_head-sized product, where launch and ramp no longer dominate: 139 MB per launch
        n = 32000
        copies = [_dev_weights(P, torch, F.Q8_0, n, k, 1100 + i) for i in range(4)]  # 557 MB > 4x L2
        y = torch.empty((1, n), device="cuda")
        torch.cuda.synchronize()
        with P.capture() as cap:
            for w in copies:
                P.gemm_quant_nt_dev(w, x, y, 1, mode=P.MODE_INT8)
        ms = _timed(P, torch, cap.graph.launch, max(args.steps // 10, 5), 3) / len(copies)
        nbytes = n * (k // 32 * 34) + 4 * k + 4 * n
        out.append({"workload": "Q8_0 GEMV 32000x4096 batch 1 (4 rotated copies)", "us_per_launch": round(ms * 1e3, 3),
                    "GBps": round(nbytes / ms / 1e6, 1), "frac_of_measured_hbm": round(nbytes / ms / 1e6 / peak_hbm, 4)})
    if args.workload in ("prefill", "all"):
        n, k = 14336, 4096
        w = _dev_weights(P, torch, F.Q4_K, n, k, 1200)
        for m in (512, 2048):
            a = torch.randn((m, k), generator=g, device="cuda")
            c = torch.empty((m, n), device="cuda")
            torch.cuda.synchronize()
            ms = _timed(P, torch, lambda: P.gemm_quant_nt_dev(w, a, c, m, mode=P.MODE_TENSOR), max(args.steps // 10, 5), 3)
            tf = 2.0 * m * n * k / ms / 1e9
            out.append({"workload": f"Q4_K prefill GEMM {m}x{n}x{k} (bf16 tcgen05, f32 out, f32->bf16 activation pass included)",
                        "ms": round(ms, 4), "TFLOPS": round(tf, 1), "frac_of_measured_bf16_burst": round(tf / 1621.7, 4),
                        "frac_of_nominal_2250": round(tf / 2250.0, 4)})
    if args.workload in ("moe", "all"):
        hidden, ffn, E, topk = 2048, 768, 128, 8
        gate = _dev_weights(P, torch, F.Q5_K, ffn, hidden, 1300, E)
        up = _dev_weights(P, torch, F.Q5_K, ffn, hidden, 1301, E)
        down = _dev_weights(P, torch, F.Q5_K, hidden, ffn, 1302, E)
        for T in (1, 8, 64, 1024):
            # 16 routing variants are rotated so a decode step does not find the previous step's experts in L2
            # (16 x 8 expert slots at T = 1 touch ~80 distinct experts, ~260 MB); one CUDA graph per variant, as a
            # decode loop would replay it
            variants = 16 if T <= 64 else 2
            xs_ = [torch.randn((T, hidden), generator=g, device="cuda") for _ in range(variants)]
            lgs = [torch.randn((T, E), generator=g, device="cuda") for _ in range(variants)]
            sel = torch.empty((T, topk), dtype=torch.int32, device="cuda")
            wts = torch.empty((T, topk), device="cuda")
            o = torch.empty((T, hidden), device="cuda")
            torch.cuda.synchronize()

            def layer(i):
                P.router_topk_dev(lgs[i], T, E, topk, True, sel, wts)
                P.moe_layer_dev(gate, up, down, xs_[i], T, topk, sel, wts, o)

            for i in range(variants):
                layer(i)
            P.synchronize()
            graphs = []
            for i in range(variants):
                with P.capture() as cap:
                    layer(i)
                graphs.append(cap.graph)
            it = [0]

            def step():
                graphs[it[0] % variants].launch()
                it[0] += 1

            ms = _timed(P, torch, step, max(args.steps // 2, 16), 3)
            out.append({"workload": f"Q5_K MoE layer hidden 2048 ffn 768 128 experts top-8, {T} tokens (router + layer on device, "
                                    f"graph replay, {variants} routing variants rotated)",
                        "ms": round(ms, 4), "tok_per_s": round(T / ms * 1e3, 1)})
    if args.workload in ("ternary", "all"):
        n = k = 8192
        rng = np.random.default_rng(4000)
        trits = rng.integers(-1, 2, size=(n, k)).astype(np.int8)
        scales = np.abs(rng.standard_normal((n, k // 256)) * 0.02).astype(np.float32)
        w = P.Weights.upload(F.TQ2_0, F.pack_ptqtp_plane(trits, scales), n, k)
        for m in (1, 256):
            a = torch.randn((m, k), generator=g, device="cuda")
            c = torch.empty((m, n), device="cuda")
            torch.cuda.synchronize()
            ms = _timed(P, torch, lambda: P.gemm_quant_nt_dev(w, a, c, m, mode=P.MODE_INT8), max(args.steps // 10, 5), 3)
            nbytes = n * (k // 256 * 66) + 4 * m * (k + n)
            out.append({"workload": f"TQ2_0 (PTQTP plane) {m}x{n}x{k}, int8 path (weights fit L2: warm-L2 figure)", "ms": round(ms, 4),
                        "GBps": round(nbytes / ms / 1e6, 1), "TFLOPS": round(2.0 * m * n * k / ms / 1e9, 2)})
            if m > 16:  # the automatic mode: bf16 tensor cores for prefill-sized batches
                ms = _timed(P, torch, lambda: P.gemm_quant_nt_dev(w, a, c, m, mode=P.MODE_AUTO), max(args.steps // 10, 5), 3)
                out.append({"workload": f"TQ2_0 (PTQTP plane) {m}x{n}x{k}, tcgen05 path (bf16 operands)", "ms": round(ms, 4),
                            "TFLOPS": round(2.0 * m * n * k / ms / 1e9, 2)})
    return out


def run_multi(args) -> list[dict]:
    """Multi-GPU exchange forms under torchrun: column-sharded Q4_K prefill with an NCCL all-gather,
    and the expert-parallel Q5_K MoE layer with NCCL all-to-all dispatch/combine."""
    import torch
    import torch.distributed as dist

    from fucina_b200 import formats as F
    from fucina_b200 import parallel as par
    from fucina_b200 import provider as P

    rank, world, local = dist_setup(args.gpus)
    P.init(local)
    ext = torch.cuda.ExternalStream(P.stream_ptr())
    out = []
    steps = max(args.steps // 10, 5)

    def timed(fn) -> float:
        for _ in range(3):
            fn()
        barrier(world)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(ext):
            e0.record()
            for _ in range(steps):
                fn()
            e1.record()
        P.synchronize()
        torch.cuda.synchronize()
        barrier(world)
        return max_over_ranks(e0.elapsed_time(e1), world) / steps

    if args.workload in ("tp_prefill", "multi"):
        n, k = 14336, 4096
        lo, hi = par.shard_rows(n, world, rank)
        w = _dev_weights(P, torch, F.Q4_K, hi - lo, k, 1200 + rank)
        for m in (512, 2048):
            g = torch.Generator(device="cuda").manual_seed(2200 + m)
            a = torch.randn((m, k), generator=g, device="cuda")
            y_local = torch.empty((m, hi - lo), device="cuda")
            torch.cuda.synchronize()

            def gemm(t):
                P.gemm_quant_nt_dev(w, t, y_local, m, mode=P.MODE_TENSOR)
                return y_local

            lin = par.ColumnShardedLinear(n, gemm) if world > 1 else None

            def step():
                with torch.cuda.stream(ext):
                    if lin is not None:
                        lin.forward(a)
                    else:
                        gemm(a)

            ms = timed(step)
            ms_compute = timed(lambda: gemm(a))
            tf = 2.0 * m * n * k / ms / 1e9
            out.append({"workload": f"Q4_K prefill {m}x{n}x{k}, columns sharded over {world} GPU(s), f32 all-gather (NCCL)",
                        "n_gpus": world, "ms": round(ms, 4), "ms_compute_only": round(ms_compute, 4), "TFLOPS_total": round(tf, 1),
                        "gathered_MB_per_rank": round(m * n * 4 * (world - 1) / world / 1e6, 1)})
    if args.workload in ("ep_moe", "multi"):
        hidden, ffn, E, topk = 2048, 768, 128, 8
        per = E // world
        gate = _dev_weights(P, torch, F.Q5_K, ffn, hidden, 1300 + rank, per)
        up = _dev_weights(P, torch, F.Q5_K, ffn, hidden, 1400 + rank, per)
        down = _dev_weights(P, torch, F.Q5_K, hidden, ffn, 1500 + rank, per)

        def ffn_rows(rows, local_expert):
            R = rows.shape[0]
            ones = torch.ones((R,), device="cuda")
            o = torch.empty_like(rows)
            P.moe_layer_dev(gate, up, down, rows, R, 1, local_expert, ones, o)
            return o

        moe = par.ExpertParallelMoE(E, topk, ffn_rows) if world > 1 else None

        def partial_rows(x_all, sel_all, w_all):
            o = torch.empty_like(x_all)
            P.moe_layer_ep_dev(gate, up, down, x_all, x_all.shape[0], topk, sel_all, w_all, rank * per, o)
            return o

        # strong scaling (64 and 1024 tokens in total) and weak scaling (1024 tokens per GPU)
        cases = [(64, "strong"), (1024, "strong")] + ([(1024 * world, "weak")] if world > 1 else [])
        for T_total, scaling in cases:
            T = T_total // world
            g = torch.Generator(device="cuda").manual_seed(3000 + 10 * rank + T_total)
            x = torch.randn((T, hidden), generator=g, device="cuda")
            logits = torch.randn((T, E), generator=g, device="cuda")
            sel = torch.empty((T, topk), dtype=torch.int32, device="cuda")
            wts = torch.empty((T, topk), device="cuda")
            o1 = torch.empty((T, hidden), device="cuda")
            torch.cuda.synchronize()
            forms = ["single GPU"] if moe is None else ["NCCL all-to-all dispatch/combine", "NCCL all-gather + reduce-scatter of partial sums",
                                                        "NCCL all-gather + reduce-scatter of partial sums, 2 token chunks pipelined",
                                                        "NCCL all-gather (bf16 tokens) + reduce-scatter of partial sums",
                                                        "NCCL all-gather (bf16 tokens) + reduce-scatter of partial sums, 2 token chunks pipelined"]
            if T % 2 or T < 512:   # decode-sized batches keep f32 tokens (the int8 arm quantises them) and one exchange
                forms = forms[:2]
            for form in forms:
                def step():
                    with torch.cuda.stream(ext):
                        P.router_topk_dev(logits, T, E, topk, True, sel, wts)
                        if moe is None:
                            P.moe_layer_dev(gate, up, down, x, T, topk, sel, wts, o1)
                        elif form.startswith("NCCL all-to-all"):
                            moe.forward(x, sel, wts)
                        else:
                            moe.forward_gathered(x, sel, wts, partial_rows, chunks=2 if form.endswith("pipelined") else 1,
                                                 exchange_dtype=torch.bfloat16 if "bf16" in form else None)

                ms = timed(step)
                out.append({"workload": f"Q5_K MoE layer (hidden 2048, ffn 768, 128 experts, top-8), {T_total} tokens over {world} GPU(s), "
                                        f"{per} experts per GPU, {form}", "scaling": scaling, "n_gpus": world, "ms": round(ms, 4),
                            "tok_per_s_total": round(T_total / ms * 1e3, 1)})
    if world > 1:
        dist.destroy_process_group()
    return out if rank == 0 else []


def run_profile_tc(args) -> dict:
    """A small case of the tensor-core prefill kernel for profiler captures: Q4_K 512 x 4096 x 4096."""
    import torch

    from fucina_b200 import formats as F
    from fucina_b200 import provider as P

    P.init(0)
    m, n, k = 512, 4096, 4096
    w = _dev_weights(P, torch, F.Q4_K, n, k, 91)
    g = torch.Generator(device="cuda").manual_seed(92)
    a = torch.randn((m, k), generator=g, device="cuda")
    c = torch.empty((m, n), device="cuda")
    torch.cuda.synchronize()
    ms = _timed(P, torch, lambda: P.gemm_quant_nt_dev(w, a, c, m, mode=P.MODE_TENSOR), args.steps, args.warmup)
    return {"workload": f"profile case: Q4_K prefill {m}x{n}x{k} tcgen05", "ms": round(ms, 4),
            "TFLOPS": round(2.0 * m * n * k / ms / 1e9, 1)}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--workload", default="stack", choices=["stack", "profile", "profile_q8", "profile_tc", "profile_moe", "q8_0", "prefill", "moe", "ternary", "all",
                                                                "tp_prefill", "ep_moe", "multi"])
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--batch", type=int, default=1, help="activation rows per product of the decode stack (1, 4 or 16)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    # Libraries (NCCL prints its version banner) may write to stdout; the contract is ONE JSON line
    # there. Everything else goes to stderr: stdout is parked and only _emit writes to it.
    sys.stdout.flush()
    real_stdout = os.dup(1)
    os.dup2(2, 1)

    def print(*a, **kw):  # noqa: A001 - shadows the builtin on purpose inside main
        os.write(real_stdout, (" ".join(str(x) for x in a) + "\n").encode())

    if args.workload == "profile":
        print(json.dumps(run_profile_case(args)), flush=True)
        return
    if args.workload == "profile_tc":
        print(json.dumps(run_profile_tc(args)), flush=True)
        return
    if args.workload == "profile_moe":
        print(json.dumps(run_profile_moe(args)), flush=True)
        return
    if args.workload == "profile_q8":
        print(json.dumps(run_profile_q8(args)), flush=True)
        return
    if args.workload in ("tp_prefill", "ep_moe", "multi"):
        for line in run_multi(args):
            print(json.dumps(line), flush=True)
        return
    if args.workload != "stack":
        for line in run_extra(args):
            print(json.dumps(line), flush=True)
        return
    out = run_reference(args) if args.impl == "reference" else run_ours(args)
    if out:
        print(json.dumps(out), flush=True)
    if int(os.environ.get("WORLD_SIZE", "1")) > 1 and args.impl == "ours":
        import torch.distributed as dist

        dist.destroy_process_group()


if __name__ == "__main__":
    main()
