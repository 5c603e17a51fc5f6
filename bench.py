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

`sub`     one record per other configuration of the metric, measured in the same
          run: Q8_0 GEMV 4096^2 (GB/s), Q4_K prefill 512 / 2048 x 14336 x 4096
          (TFLOP/s), the Q5_K MoE layer at 1 / 64 / 1024 tokens (tok/s) and the
          ternary 8192^2 products, each with its roofline fraction and its own
          CPU baseline (all host threads and one thread).

The timed region of `value` is R repeats of the K-step sequence between one
pair of CUDA events (R chosen so that the region lasts about half a second and
the clock sampler sees it); ms_per_step = elapsed / (R * K).

With --gpus N > 1 every rank serves its own decode stream from its own weight
replica (weak scaling, no collective on the data path); time is the max over
ranks. `sub` then carries the two exchange forms instead: the expert-parallel
MoE layer (weak: 1024 tokens per GPU; strong: 1024 in total) and the
column-sharded prefill with its all-gather.
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


def measured_tflops() -> tuple[float, float, str]:
    """(burst, sustained) dense bf16 TFLOP/s of this pool's B200s, and where the numbers come from."""
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            d = json.load(open(p))
            return float(d["bf16_tflops"]), float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "measured"
        except Exception:
            pass
    return 1590.0, 1400.0, "fallback"


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

        import datetime

        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        # a bounded group timeout: a rank that failed must end the others' next collective, not hang them
        dist.init_process_group("nccl", device_id=torch.device("cuda", local), timeout=datetime.timedelta(seconds=300))
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

    def product_graphs(i: int):
        """Product i of the stack alone: one launch per weight copy, and the cycle over all copies."""
        singles = []
        for c in range(n_copies):
            with P.capture() as cap:
                P.gemm_quant_nt_dev(stacks[c].weights[i], xs[i], ys[i], batch, mode=P.MODE_INT8)
            singles.append(cap.graph)
        with P.capture() as cap:
            for c in range(n_copies):
                P.gemm_quant_nt_dev(stacks[c].weights[i], xs[i], ys[i], batch, mode=P.MODE_INT8)
        return cap.graph, singles

    def timed_graphs(cycle, graphs, steps: int, repeats: int = 1) -> float:
        """milliseconds of `repeats` x (exactly `steps` steps: whole cycles of n_copies steps, then single-step graphs)."""
        barrier(world)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(ext):
            e0.record()
            for _ in range(repeats):
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
        step_cycle.launch()
    P.synchronize()

    # ---- value: resident inputs, CUDA events on the library stream ----
    # R repeats of the K-step sequence inside one timed region of about half a second, so the clock
    # sampler (100 ms period) describes the region that was timed
    est = timed_graphs(step_cycle, step_graphs, args.steps) / args.steps  # ms per step, first estimate
    repeats = max(1, min(200000, int(500.0 / max(est * args.steps, 1e-3))))
    with ClockSampler(local) as clk:
        ms = timed_graphs(step_cycle, step_graphs, args.steps, repeats)
    # one decode kernel per product with the activation quantisation fused in (batch <= 4); wider batches
    # quantise in a kernel of their own first
    launches = repeats * args.steps * len(STACK_N) * (1 if batch <= 4 else 2)
    bytes_step = stack_bytes(batch)
    ms_step = ms / (repeats * args.steps)
    value = world * bytes_step / (ms_step * 1e-3) / 1e9

    # ---- roofline: each product alone, back-to-back launches over the rotated copies; the dominant one is the headline kernel ----
    peak, peak_src = measured_peaks()
    big = max(range(len(STACK_N)), key=lambda i: STACK_N[i])
    per_product = []
    k_n = max(args.steps, n_copies)
    for i, n in enumerate(STACK_N):
        cyc, singles = product_graphs(i)
        for _ in range(3):
            cyc.launch()
        P.synchronize()
        one = timed_graphs(cyc, singles, k_n) / k_n
        reps = max(1, min(200000, int(100.0 / max(one * k_n, 1e-3))))  # about 0.1 s per product
        k_ms = timed_graphs(cyc, singles, k_n, reps) / (reps * k_n)
        nbytes = n * ROW_BYTES + batch * K * 4 + batch * n * 4
        per_product.append({"n": n, "k": K, "us_per_launch": round(k_ms * 1e3, 3), "bytes_per_launch": nbytes,
                            "GBps": round(nbytes / (k_ms * 1e-3) / 1e9, 1), "frac": round(nbytes / (k_ms * 1e-3) / 1e9 / peak, 4),
                            "launches_timed": reps * k_n})
        del cyc, singles
    dom = per_product[big]
    roofline = {"bound": "hbm", "achieved": dom["GBps"], "peak": peak, "unit": "GB/s", "frac": dom["frac"],
                # dram__bytes_read + dram__bytes_write of one profiler capture of the same kernel on a 65536-row
                # matrix (151.31 MB + 3.46 MB), scaled to this launch by rows (traffic is proportional to rows)
                "traffic": int((151_309_056 + 3_462_656) * STACK_N[big] / 65536),
                "traffic_source": "ncu capture of a 65536 x 4096 case, scaled by rows",
                "kernel": f"decode_rows_kernel<Q4_K, MB={batch}, fused act-quant> on 32000x4096",
                "peak_source": peak_src, "launches_timed": dom["launches_timed"],
                "timing": "CUDA events around back-to-back launches (graph replay, consecutive launches overlap by programmatic dependent launch)",
                "us_per_launch": dom["us_per_launch"], "bytes_per_launch": dom["bytes_per_launch"],
                "frac_of_8TBs": round(dom["GBps"] / 8000.0, 4), "per_product": per_product}

    # ---- e2e: blocking C-ABI call, host buffers, resident weights ----
    host_x = [x.cpu().numpy() for x in xs]
    host_y = [np.empty((batch, n), np.float32) for n in STACK_N]
    # the caller's activation and result storage is registered once, as the reference registers tensor storage
    # for its lifetime (src/backend/cuda.zig:1047-1082): DMA reads it and the kernels write it without a bounce
    for arr in host_x + host_y:
        P.host_register(arr)

    def step_host(i: int):
        st = stacks[i % n_copies]
        for hw, x, y, n in zip(st.host, host_x, host_y, STACK_N):
            P.gemm_quant_nt(Q4_K, hw, x, n, cacheable=True, out=y)

    e2e_steps = max(args.steps, 200)  # a step is ~0.1 ms of wall clock: enough of them for a steady figure
    for i in range(max(args.warmup, n_copies)):  # first touch adopts each copy's weights
        step_host(i)
    barrier(world)
    t0 = time.perf_counter()
    for i in range(e2e_steps):
        step_host(i)
    P.synchronize()
    e2e_s = max_over_ranks(time.perf_counter() - t0, world)
    barrier(world)
    blocking = {"value": round(world * bytes_step * e2e_steps / e2e_s / 1e9, 2), "unit": "GB/s", "ms_per_step": round(e2e_s / e2e_steps * 1e3, 4),
                "call": "fq_gemm_quant_nt (blocking), one call per product, from Python through ctypes"}

    # the same step through the asynchronous entry (the reference's gemmQuantNtAsync + Work.finish): the
    # four products of a step are submitted back to back and finished afterwards, so uploads, kernels and
    # downloads of different products overlap
    # the argument conversion of the four calls is done once per weight copy (provider.PreparedGemmAsync): what is
    # left between two C-ABI calls is one foreign-function call of the interpreter
    prepared = [[P.PreparedGemmAsync(Q4_K, hw, x, n, batch, K, out=y) for hw, x, y, n in zip(st.host, host_x, host_y, STACK_N)]
                for st in stacks]

    def step_host_async(i: int):
        calls = prepared[i % n_copies]
        for c in calls:
            c.submit()
        for c in calls:
            c.finish()

    for i in range(max(args.warmup, n_copies)):
        step_host_async(i)
    barrier(world)
    t0 = time.perf_counter()
    for i in range(e2e_steps):
        step_host_async(i)
    P.synchronize()
    async_s = max_over_ranks(time.perf_counter() - t0, world)
    barrier(world)
    queued = {"value": round(world * bytes_step * e2e_steps / async_s / 1e9, 2), "unit": "GB/s", "ms_per_step": round(async_s / e2e_steps * 1e3, 4),
              "call": "fq_gemm_quant_nt_async x4, then fq_work_finish x4 (the reference's own first choice, exec/quant_matmul.zig:959-1051), "
                      "from Python through ctypes, arguments converted once per weight copy"}
    # the headline end-to-end figure is the faster of the two public forms; both are reported
    best = queued if queued["value"] > blocking["value"] else blocking
    e2e = {"value": best["value"], "unit": "GB/s", "h2d_bytes_per_step": len(STACK_N) * batch * K * 4,
           "d2h_bytes_per_step": sum(STACK_N) * batch * 4, "ms_per_step": best["ms_per_step"], "steps_timed": e2e_steps,
           "timing": "wall clock between device syncs; host activation and result storage registered once (fq_host_register)",
           "call": best["call"], "blocking": blocking, "async_queue": queued}
    for arr in host_x + host_y:
        P.host_unregister(arr)
    if rank == 0:
        native = native_e2e(batch)
        if native:
            e2e["native_caller"] = native

    out = {
        "metric": "quant GEMV HBM GB/s", "value": round(value, 1), "unit": "GB/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(ms_step, 5), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "int8xq4 -> f32", "data": "synthetic",
        "config": {"workload": f"Q4_K decode GEMV stack, batch {batch}, K=4096 -> N in {{4096,11008,4096,32000}}",
                   "bytes_per_step": bytes_step, "weight_copies_rotated": n_copies,
                   "l2_policy": f"inputs larger than L2: {n_copies} distinct weight copies ({n_copies * bytes_step >> 20} MiB) rotated",
                   "timed_region": f"{repeats} repeats of the {args.steps}-step sequence between one pair of CUDA events ({ms:.0f} ms)",
                   "parallelism": f"dp{world} replicas" if world > 1 else "single GPU"},
        "frac_of_8TBs": round(value / world / 8000.0, 4),
        "roofline": roofline, "e2e": e2e, "gpu_launches": launches, "clocks": clk.summary(),
    }
    # ---- the other configurations of the metric, in the same line ----
    del step_graphs, step_cycle
    host_stack = stacks[0].host
    stacks = None
    torch.cuda.empty_cache()
    if not args.no_sub:
        want_cpu = rank == 0 and world == 1 and not args.no_cpu
        out["sub"] = sub_records(args, P, torch, rank, world, local, want_cpu)
    if rank == 0 and world == 1 and not args.no_cpu:
        out["cpu_baseline"] = cpu_baseline(host_stack, host_x, budget_s=8.0)
    return out if rank == 0 else {}


def native_e2e(batch: int) -> dict | None:
    """The same blocking host-buffer step from a C caller (no interpreter between the calls): the harness built
    beside the library, run as a child process. Separates the library's per-call cost from Python's."""
    exe = os.path.join(ROOT, "fucina_b200", "lib", "e2e_harness")
    if not os.path.exists(exe):
        return None
    try:
        r = subprocess.run([exe, str(batch)], capture_output=True, text=True, timeout=120,
                           env={**os.environ, "CUDA_VISIBLE_DEVICES": os.environ.get("CUDA_VISIBLE_DEVICES", "")} if os.environ.get("CUDA_VISIBLE_DEVICES") else None)
        line = [ln for ln in r.stdout.splitlines() if ln.startswith("{")]
        return json.loads(line[-1]) if line else {"error": (r.stderr or r.stdout)[-200:]}
    except Exception as e:  # noqa: BLE001 - the harness is information, never fatal
        return {"error": str(e)[:200]}


def _cpu_time(fn, budget_s: float, max_calls: int = 100000) -> tuple[float, int]:
    """seconds per call of fn() over about budget_s of wall clock (at least one call)."""
    fn()
    t0 = time.perf_counter()
    calls = 0
    while True:
        fn()
        calls += 1
        dt = time.perf_counter() - t0
        if dt > budget_s or calls >= max_calls:
            return dt / calls, calls


def _cpu_stack_step(host_w, host_x):
    """The CPU arm to time for the Q4_K stack: the reference's load-time eight-row repack (BlockQ4_Kx8,
    src/backend/quant/q4_k.zig:127-192, :1733-1782) where this host can run it, else the compact row kernels;
    whichever is faster on a trial pass, as the reference's dispatch would keep the faster one. Returns (step, label)."""
    import oracle

    def compact():
        for w, x in zip(host_w, host_x):
            oracle.matmul_fast(Q4_K, w, x)

    label = "AVX2 compact block dots" if oracle.has_simd(Q4_K) else "scalar block dots"
    packs = [oracle.PackedRows.pack(Q4_K, w, K) for w in host_w]
    if any(p is None for p in packs):
        return compact, label

    def packed():
        for p, x in zip(packs, host_x):
            p.matmul(x)

    t_c, _ = _cpu_time(compact, 0.3, 50)
    t_p, _ = _cpu_time(packed, 0.3, 50)
    return (packed, "AVX2 eight-row packs (BlockQ4_Kx8, packed once before the timed region)") if t_p < t_c else (compact, label)


def cpu_baseline(host_w, host_x, budget_s: float) -> dict:
    """The CPU restatement of the reference kernels (activations to Q8_K, Q4_K block dots on the fastest arm,
    output columns split over the host threads) on one stack copy, a few passes; all host threads, then one."""
    import oracle

    bytes_step = stack_bytes(1)
    cores = oracle.set_threads(0)
    step, arm = _cpu_stack_step(host_w, host_x)

    sec, passes = _cpu_time(step, budget_s, 5000)
    oracle.set_threads(1)
    sec1, passes1 = _cpu_time(step, min(budget_s, 3.0), 5000)
    oracle.set_threads(0)
    return {"value": round(bytes_step / sec / 1e9, 3), "unit": "GB/s", "cores": cores, "kind": "port",
            "sample": f"{passes} pass(es) of the full stack (4 products, batch 1), {sec * passes:.1f} s, " + arm,
            "ms_per_step": round(sec * 1e3, 3),
            "single_thread": {"value": round(bytes_step / sec1 / 1e9, 3), "unit": "GB/s", "ms_per_step": round(sec1 * 1e3, 3), "passes": passes1}}


def run_reference(args) -> dict:
    """The reference's CPU path for the same workload and the same bytes per step: its Zig kernels cannot be
    built here (no Zig toolchain), so the timed code is their C++ restatement in oracle/ (SIMD block dots,
    columns split over the host threads as QuantizedRhsParallel does). The worker count is set explicitly:
    launchers such as torchrun export OMP_NUM_THREADS=1."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return {}
    import oracle

    cores = oracle.set_threads(0)
    rng = np.random.default_rng(1100)
    # seeded N(0,0.02) weights through the restated reference encoder, the full stack
    ws = [oracle.quantize_rows(Q4_K, (rng.standard_normal((n, K)) * 0.02).astype(np.float32)) for n in STACK_N]
    xs = [rng.standard_normal((1, K)).astype(np.float32) for _ in STACK_N]
    bytes_step = stack_bytes(1)

    step, arm = _cpu_stack_step(ws, xs)

    for _ in range(args.warmup):
        step()
    # R repeats of the K-step sequence, at least a second of wall clock
    t0 = time.perf_counter()
    step()
    one = time.perf_counter() - t0
    repeats = max(1, int(1.0 / max(one * args.steps, 1e-6)) + 1)
    t0 = time.perf_counter()
    for _ in range(repeats * args.steps):
        step()
    dt = time.perf_counter() - t0
    n_steps = repeats * args.steps
    value = round(bytes_step * n_steps / dt / 1e9, 3)
    sample = f"the full stack (4 products, batch 1) per step, {repeats} x {args.steps} steps, {dt:.1f} s, {cores} threads, " + arm
    return {
        "impl": "reference", "metric": "quant GEMV HBM GB/s", "value": value, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(dt / n_steps * 1e3, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8xq4 -> f32", "data": "synthetic",
        "config": {"workload": "Q4_K decode GEMV stack, batch 1, K=4096 -> N in {4096,11008,4096,32000}",
                   "bytes_per_step": bytes_step, "threads": cores,
                   "note": "CPU restatement of the reference kernels; Zig toolchain absent"},
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
    hidden, ffn, n_expert, top_k, seq = 2048, 768, 128, 8, max(1, args.tokens)
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
    return {"workload": f"profile case: Q5_K MoE layer 2048/768, 128 experts, top-8, {seq} tokens (plain launches)", "ms": round(ms, 4),
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


def _dev_weights(P, torch, fmt: int, n: int, k: int, seed: int, n_mats: int = 1, keep_host: bool = False):
    """Seeded N(0, 0.02) f32 rows through the library's device encoder -> device-resident weights; with keep_host
    the raw GGUF bytes are also kept on the host (`.host`, [n_mats * n, row_bytes]) for the CPU baseline."""
    from fucina_b200 import formats as F

    g = torch.Generator(device="cuda").manual_seed(seed)
    rb = F.row_bytes(fmt, k)
    blocks = torch.empty(n_mats * n * rb, dtype=torch.uint8, device="cuda")
    for e in range(n_mats):  # one matrix at a time keeps the f32 staging small
        w = torch.randn((n, k), generator=g, device="cuda", dtype=torch.float32) * 0.02
        torch.cuda.synchronize()
        P.quantize_rows_dev(fmt, w, n, k, blocks[e * n * rb:(e + 1) * n * rb])
        P.synchronize()
    wt = P.Weights.from_device(fmt, blocks, n, k, n_mats)
    if keep_host:
        wt.host = blocks.cpu().numpy().reshape(n_mats * n, rb)
    return wt


# ----------------------------------------------------------------------------------------------
# The other configurations of the metric: one record each inside the default line's `sub` list.
# ----------------------------------------------------------------------------------------------
def _graph_ms(P, torch, graphs, target_ms: float = 150.0) -> float:
    """milliseconds per launch over the rotated graphs, timed for about target_ms on the library stream."""
    it = [0]

    def step():
        graphs[it[0] % len(graphs)].launch()
        it[0] += 1

    one = _timed(P, torch, step, len(graphs), 3)
    steps = max(len(graphs), min(200000, int(target_ms / max(one, 1e-4))))
    return _timed(P, torch, step, steps, 0)


def sub_q8_0(args, P, torch, want_cpu: bool) -> list[dict]:
    """Q8_0 GEMV 4096 x 4096, batch 1 (the bench/q8gemv.zig shape): 30 rotated weight copies (535 MB > 4x L2)."""
    import oracle
    from fucina_b200 import formats as F

    n = k = 4096
    peak, src = measured_peaks()
    host = oracle.quantize_rows(F.Q8_0, (np.random.default_rng(1000).standard_normal((n, k)) * 0.02).astype(np.float32))
    copies = [_dev_weights(P, torch, F.Q8_0, n, k, 1001 + i) for i in range(30)]
    g = torch.Generator(device="cuda").manual_seed(2000)
    x = torch.randn((1, k), generator=g, device="cuda")
    y = torch.empty((1, n), device="cuda")
    torch.cuda.synchronize()
    with P.capture() as cap:
        for w in copies:
            P.gemm_quant_nt_dev(w, x, y, 1, mode=P.MODE_INT8)
    ms = _graph_ms(P, torch, [cap.graph]) / len(copies)
    nbytes = n * (k // 32 * 34) + 4 * k + 4 * n
    gbs = nbytes / ms / 1e6
    rec = {"workload": "Q8_0 GEMV 4096x4096 batch 1 (30 rotated weight copies, graph replay)", "metric": "quant GEMV HBM GB/s",
           "value": round(gbs, 1), "unit": "GB/s", "us_per_launch": round(ms * 1e3, 3), "bytes_per_launch": nbytes,
           "roofline": {"bound": "hbm", "achieved": round(gbs, 1), "peak": peak, "unit": "GB/s", "frac": round(gbs / peak, 4),
                        "peak_source": src, "frac_of_8TBs": round(gbs / 8000.0, 4), "kernel": "decode_rows_kernel<Q8_0, MB=1>"}}
    if want_cpu:
        xh = x.cpu().numpy()
        cores = oracle.set_threads(0)
        fn, arm = (lambda: oracle.matmul_fast(F.Q8_0, host, xh)), ("AVX2 block dots" if oracle.has_simd(F.Q8_0) else "scalar")
        pk = oracle.PackedRows.pack(F.Q8_0, host, k)  # the reference's four-row pack (BlockQ8_0x4), kept if it is the faster arm here
        if pk is not None and _cpu_time(lambda: pk.matmul(xh), 0.2, 50)[0] < _cpu_time(fn, 0.2, 50)[0]:
            fn, arm = (lambda: pk.matmul(xh)), "AVX2 four-row packs (BlockQ8_0x4)"
        sec, calls = _cpu_time(fn, 1.5)
        oracle.set_threads(1)
        sec1, _ = _cpu_time(fn, 1.0)
        oracle.set_threads(0)
        rec["cpu_baseline"] = {"value": round(nbytes / sec / 1e9, 2), "unit": "GB/s", "cores": cores, "kind": "port",
                               "sample": f"{calls} products, {sec * calls:.1f} s, " + arm,
                               "single_thread": {"value": round(nbytes / sec1 / 1e9, 2), "unit": "GB/s"}}
    return [rec]


def sub_q6_k(args, P, torch, want_cpu: bool) -> list[dict]:
    """Q6_K decode product 32000 x 4096, batch 1: the output tensor of a mixed K-quant file (its largest single matrix);
    six rotated weight copies (645 MB > 4x L2) inside one graph."""
    import oracle
    from fucina_b200 import formats as F

    n, k = 32000, 4096
    peak, src = measured_peaks()
    copies = [_dev_weights(P, torch, F.Q6_K, n, k, 1600 + i) for i in range(6)]
    g = torch.Generator(device="cuda").manual_seed(2600)
    x = torch.randn((1, k), generator=g, device="cuda")
    y = torch.empty((1, n), device="cuda")
    P.gemm_quant_nt_dev(copies[0], x, y, 1, mode=P.MODE_INT8)
    P.synchronize()
    with P.capture() as cap:
        for w in copies:
            P.gemm_quant_nt_dev(w, x, y, 1, mode=P.MODE_INT8)
    ms = _graph_ms(P, torch, [cap.graph]) / len(copies)
    nbytes = n * (k // 256 * 210) + 4 * k + 4 * n
    gbs = nbytes / ms / 1e6
    rec = {"workload": "Q6_K decode product 32000x4096 batch 1 (6 rotated weight copies, graph replay)", "metric": "quant GEMV HBM GB/s",
           "value": round(gbs, 1), "unit": "GB/s", "us_per_launch": round(ms * 1e3, 3), "bytes_per_launch": nbytes,
           "roofline": {"bound": "hbm", "achieved": round(gbs, 1), "peak": peak, "unit": "GB/s", "frac": round(gbs / peak, 4),
                        "peak_source": src, "frac_of_8TBs": round(gbs / 8000.0, 4), "kernel": "decode_rows_kernel<Q6_K, MB=1, 16 warps>"}}
    if want_cpu:
        host = oracle.quantize_rows(F.Q6_K, (np.random.default_rng(1600).standard_normal((2048, k)) * 0.02).astype(np.float32))
        xh = x.cpu().numpy()
        cores = oracle.set_threads(0)
        fn, arm = (lambda: oracle.matmul_fast(F.Q6_K, host, xh)), ("AVX2 block dots" if oracle.has_simd(F.Q6_K) else "scalar block dots")
        pk = oracle.PackedRows.pack(F.Q6_K, host, k)  # the reference's four-row pack (BlockQ6_Kx4), kept if it is the faster arm here
        if pk is not None and _cpu_time(lambda: pk.matmul(xh), 0.2, 50)[0] < _cpu_time(fn, 0.2, 50)[0]:
            fn, arm = (lambda: pk.matmul(xh)), "AVX2 four-row packs (BlockQ6_Kx4)"
        sec, calls = _cpu_time(fn, 1.0)
        rec["cpu_baseline"] = {"value": round(host.nbytes / sec / 1e9, 2), "unit": "GB/s", "cores": cores, "kind": "port",
                               "sample": f"2048 of the 32000 weight rows, {calls} products, {sec * calls:.1f} s, " + arm}
    return [rec]


def sub_prefill(args, P, torch, want_cpu: bool) -> list[dict]:
    """Q4_K prefill GEMM, M in {512, 2048} x N 14336 x K 4096: bf16 tcgen05 MMA, f32 accumulate and output."""
    import oracle
    from fucina_b200 import formats as F

    n, k = 14336, 4096
    burst, sustained, src = measured_tflops()
    w = _dev_weights(P, torch, F.Q4_K, n, k, 1200)
    g = torch.Generator(device="cuda").manual_seed(2200)
    recs = []
    for m in (512, 2048):
        a = torch.randn((m, k), generator=g, device="cuda").to(torch.bfloat16).to(torch.float32)  # bf16 activations of the config
        c = torch.empty((m, n), device="cuda")
        torch.cuda.synchronize()
        fn = lambda: P.gemm_quant_nt_dev(w, a, c, m, mode=P.MODE_TENSOR)  # noqa: E731
        one = _timed(P, torch, fn, 5, 3)
        ms = _timed(P, torch, fn, max(5, min(2000, int(150.0 / one))), 0)
        tf = 2.0 * m * n * k / ms / 1e9
        recs.append({"workload": f"Q4_K prefill GEMM {m}x{n}x{k} (bf16 tcgen05, f32 out; the f32->bf16 activation pass is inside the timed call)",
                     "metric": "Q4_K prefill TFLOPS", "value": round(tf, 1), "unit": "TFLOP/s", "ms": round(ms, 4),
                     "roofline": {"bound": "tensor", "achieved": round(tf, 1), "peak": burst, "unit": "TFLOP/s", "frac": round(tf / burst, 4),
                                  "peak_source": src + " (burst)", "frac_of_sustained": round(tf / sustained, 4),
                                  "frac_of_nominal_2250": round(tf / 2250.0, 4), "kernel": "gemm_tc_kernel<Q4_K, TN=256>"}})
    if want_cpu:
        # bounded sample: 32 of the activation rows against the whole matrix (the row arm of the CPU threading)
        rng = np.random.default_rng(1200)
        host = oracle.quantize_rows(F.Q4_K, (rng.standard_normal((n, k)) * 0.02).astype(np.float32))
        ah = rng.standard_normal((32, k)).astype(np.float32)
        cores = oracle.set_threads(0)
        pk, pk1 = oracle.PackedRows.pack(F.Q4_K, host, k), oracle.PackedRows.pack(F.Q4_K, host[:2048], k)
        full = (lambda: pk.matmul(ah)) if pk else (lambda: oracle.matmul_fast(F.Q4_K, host, ah))
        part = (lambda: pk1.matmul(ah)) if pk1 else (lambda: oracle.matmul_fast(F.Q4_K, host[:2048], ah))
        sec, calls = _cpu_time(full, 2.0)
        oracle.set_threads(1)
        sec1, _ = _cpu_time(part, 1.0)
        oracle.set_threads(0)
        cpu = {"value": round(2.0 * 32 * n * k / sec / 1e12, 4), "unit": "TFLOP/s", "cores": cores, "kind": "port",
               "sample": f"32 activation rows x the whole 14336 x 4096 matrix, {calls} passes, {sec * calls:.1f} s, int8 block dots"
                         + (" over eight-row packs (BlockQ4_Kx8)" if pk else ""),
               "single_thread": {"value": round(2.0 * 32 * 2048 * k / sec1 / 1e12, 4), "unit": "TFLOP/s", "sample": "32 rows x 2048 weight rows"}}
        for r in recs:
            r["cpu_baseline"] = cpu
    return recs


MOE = {"hidden": 2048, "ffn": 768, "experts": 128, "top_k": 8}


def _moe_stacks(P, torch, experts: int, seed0: int, keep_host: bool = False):
    from fucina_b200 import formats as F

    h, f = MOE["hidden"], MOE["ffn"]
    gate = _dev_weights(P, torch, F.Q5_K, f, h, seed0, experts, keep_host)
    up = _dev_weights(P, torch, F.Q5_K, f, h, seed0 + 1, experts, keep_host)
    down = _dev_weights(P, torch, F.Q5_K, h, f, seed0 + 2, experts, keep_host)
    return gate, up, down


def _moe_layer_ms(P, torch, stacks, T: int, variants: int, seed: int):
    """ms per router+layer step over `variants` rotated routings (one CUDA graph each), and the experts touched per step."""
    h, E, topk = MOE["hidden"], stacks[0].n_mats, MOE["top_k"]
    g = torch.Generator(device="cuda").manual_seed(seed)
    xs_ = [torch.randn((T, h), generator=g, device="cuda") for _ in range(variants)]
    lgs = [torch.randn((T, E), generator=g, device="cuda") for _ in range(variants)]
    sel = torch.empty((T, topk), dtype=torch.int32, device="cuda")
    wts = torch.empty((T, topk), device="cuda")
    o = torch.empty((T, h), device="cuda")
    torch.cuda.synchronize()

    def layer(i):
        P.router_topk_dev(lgs[i], T, E, topk, True, sel, wts)
        P.moe_layer_dev(*stacks, xs_[i], T, topk, sel, wts, o)

    touched = []
    for i in range(variants):
        layer(i)
        P.synchronize()
        touched.append(int(torch.unique(sel).numel()))
    graphs = []
    for i in range(variants):
        with P.capture() as cap:
            layer(i)
        graphs.append(cap.graph)
    ms = _graph_ms(P, torch, graphs)
    return ms, float(np.mean(touched))


def sub_moe(args, P, torch, want_cpu: bool) -> list[dict]:
    """Q5_K MoE expert layer (hidden 2048, ffn 768, 128 experts, top-8; router on the device, softmax top-8
    renormalised): decode batches 1 and 64 and the 1024-token prefill. Routing variants are rotated so a decode
    step does not find the previous step's experts in L2."""
    import oracle
    from fucina_b200 import formats as F

    peak, src = measured_peaks()
    burst, _, tsrc = measured_tflops()
    stacks = _moe_stacks(P, torch, MOE["experts"], 1300, keep_host=want_cpu)
    per_expert = 3 * MOE["ffn"] * (MOE["hidden"] // 256) * 176  # 3 244 032 bytes of Q5_K blocks
    flop_tok = 2.0 * MOE["top_k"] * 3 * MOE["ffn"] * MOE["hidden"]
    recs = []
    for T in (1, 64, 1024):
        ms, touched = _moe_layer_ms(P, torch, stacks, T, 16 if T <= 64 else 2, 3000 + T)
        rec = {"workload": f"Q5_K MoE layer hidden 2048 ffn 768, 128 experts, top-8, {T} token(s) (router + layer on device, graph replay, "
                           f"{16 if T <= 64 else 2} routing variants rotated)",
               "metric": "MoE layer tok/s", "value": round(T / ms * 1e3, 1), "unit": "tok/s", "ms": round(ms, 4)}
        if T <= 64:
            gbs = touched * per_expert / ms / 1e6
            rec["roofline"] = {"bound": "hbm", "achieved": round(gbs, 1), "peak": peak, "unit": "GB/s", "frac": round(gbs / peak, 4),
                               "peak_source": src, "experts_touched": round(touched, 1), "bytes": "expert weight bytes touched per step",
                               "kernel": "expert_rows_kernel<Q5_K> (gate/up fused, then down)"}
        else:
            tf = T * flop_tok / ms / 1e9
            rec["roofline"] = {"bound": "tensor", "achieved": round(tf, 1), "peak": burst, "unit": "TFLOP/s", "frac": round(tf / burst, 4),
                               "peak_source": tsrc + " (burst)", "kernel": "gemm_tc_kernel<Q5_K, TN=128> (gated pair, then down)"}
        recs.append(rec)
    if want_cpu:
        hg, hu, hd = (w.host for w in stacks)
        rng = np.random.default_rng(3000)
        cores = oracle.set_threads(0)
        # the reference's fastest arm for K-quant expert stacks: the load-time eight-row repack (BlockQ5_Kx8)
        packs = [oracle.PackedRows.pack(F.Q5_K, b, kk) for b, kk in ((hg, MOE["hidden"]), (hu, MOE["hidden"]), (hd, MOE["ffn"]))]
        if any(p is None for p in packs):
            packs = None
        for rec, T, Ts in zip(recs, (1, 64, 1024), (1, 64, 256)):
            x = rng.standard_normal((Ts, MOE["hidden"])).astype(np.float32)
            sel, wts = oracle.router_topk(rng.standard_normal((Ts, MOE["experts"])).astype(np.float32), MOE["top_k"], True)
            if packs:
                fn = lambda: oracle.moe_ffn_packed(*packs, x, sel, wts, MOE["experts"], MOE["ffn"])  # noqa: E731
            else:
                fn = lambda: oracle.moe_ffn_fast(F.Q5_K, hg, hu, hd, x, sel, wts, MOE["experts"], MOE["ffn"])  # noqa: E731
            sec, calls = _cpu_time(fn, 2.0)
            rec["cpu_baseline"] = {"value": round(Ts / sec, 1), "unit": "tok/s", "cores": cores, "kind": "port",
                                   "sample": f"{Ts} token(s) per pass" + (f" (a {Ts}-token sample of the {T})" if T != Ts else "") + f", {calls} passes, {sec * calls:.1f} s"
                                             + (", eight-row packs (BlockQ5_Kx8)" + (", pairs grouped by expert and multiplied four rows at a time" if Ts * MOE["top_k"] >= 2 * MOE["experts"] else "")
                                                if packs else "")}
            if T == 1:
                oracle.set_threads(1)
                sec1, _ = _cpu_time(fn, 1.0)
                oracle.set_threads(0)
                rec["cpu_baseline"]["single_thread"] = {"value": round(Ts / sec1, 1), "unit": "tok/s"}
    return recs


def sub_attention(args, P, torch, want_cpu: bool) -> list[dict]:
    """One decode step of streaming attention (the op next to the linear layers): 32 heads over 8 kv heads, d 128,
    f16 KV, one query row, at 8192 and at 32768 cached keys; KV copies (> L2 in total) rotated inside one graph.
    Bytes = the K and V rows read."""
    heads, kv_heads, d = 32, 8, 128
    peak, src = measured_peaks()
    g = torch.Generator(device="cuda").manual_seed(2500)
    q = torch.randn((1, heads, d), generator=g, device="cuda")
    kvmap = torch.arange(heads, device="cuda", dtype=torch.int32) // (heads // kv_heads)
    out = torch.empty((1, heads, d), device="cuda")
    scale = 1.0 / float(np.sqrt(d))
    recs = []
    for kv_seq in (8192, 32768):
        copies = [(torch.randn((kv_seq, kv_heads, d), generator=g, device="cuda").half(),
                   torch.randn((kv_seq, kv_heads, d), generator=g, device="cuda").half()) for _ in range(max(2, 6 * 8192 // kv_seq))]
        torch.cuda.synchronize()

        def step(kv):
            P.attn_fwd_dev(q, kv[0], kv[1], True, out, kvmap, 1, kv_seq, heads, kv_heads, d, kv_seq - 1, scale)

        step(copies[0])  # warm the allocator before capturing
        P.synchronize()
        with P.capture() as cap:
            for kv in copies:
                step(kv)
        ms = _graph_ms(P, torch, [cap.graph]) / len(copies)
        nbytes = 2 * kv_seq * kv_heads * d * 2
        gbs = nbytes / ms / 1e6
        rec = {"workload": f"attention decode step: 1 query row, 32 heads / 8 kv heads, d 128, {kv_seq} keys, f16 KV ({len(copies)} rotated KV copies, graph replay)",
               "metric": "attention KV GB/s", "value": round(gbs, 1), "unit": "GB/s", "us_per_step": round(ms * 1e3, 3), "bytes_per_step": nbytes,
               "roofline": {"bound": "hbm", "achieved": round(gbs, 1), "peak": peak, "unit": "GB/s", "frac": round(gbs / peak, 4), "peak_source": src,
                            "kernel": "attn_split_mma_kernel (mma.sync.m16n8k16, cp.async double-buffered tiles) + attn_merge_kernel"}}
        if want_cpu:
            qh = q.cpu().numpy()[0].astype(np.float32)
            kh, vh = copies[0][0].cpu().numpy().astype(np.float32), copies[0][1].cpu().numpy().astype(np.float32)

            def cpu():
                for h in range(heads):
                    sc = kh[:, h // (heads // kv_heads)] @ qh[h] * scale
                    pr = np.exp(sc - sc.max())
                    _ = (pr @ vh[:, h // (heads // kv_heads)]) / pr.sum()

            sec, calls = _cpu_time(cpu, 1.0)
            rec["cpu_baseline"] = {"value": round(nbytes / sec / 1e9, 2), "unit": "GB/s", "cores": os.cpu_count(), "kind": "port",
                                   "sample": f"{calls} steps, {sec * calls:.1f} s, numpy f32 (BLAS threads) over f32 copies of the same KV"}
        recs.append(rec)
        del copies, cap
        torch.cuda.empty_cache()
    return recs


def sub_ternary(args, P, torch, want_cpu: bool) -> list[dict]:
    """PTQTP ternary plane (TQ2_0, one f16 scale per 256) 8192 x 8192: batch 1 on the integer kernel over 30 rotated
    copies (519 MB > 4x L2), batch 256 on the tensor cores."""
    import oracle
    from fucina_b200 import formats as F

    n = k = 8192
    peak, src = measured_peaks()
    burst, _, tsrc = measured_tflops()
    rng = np.random.default_rng(4000)
    trits = rng.integers(-1, 2, size=(n, k)).astype(np.int8)
    scales = np.abs(rng.standard_normal((n, k // 256)) * 0.02).astype(np.float32)
    host = F.pack_ptqtp_plane(trits, scales)
    del trits
    hd = torch.from_numpy(host).cuda()
    copies = []
    for i in range(30):
        blk = torch.roll(hd, shifts=i, dims=0).contiguous()  # the same rows in another order: distinct addresses, same arithmetic
        copies.append(P.Weights.from_device(F.TQ2_0, blk, n, k))
    g = torch.Generator(device="cuda").manual_seed(2400)
    x = torch.randn((1, k), generator=g, device="cuda")
    y = torch.empty((1, n), device="cuda")
    torch.cuda.synchronize()
    with P.capture() as cap:
        for w in copies:
            P.gemm_quant_nt_dev(w, x, y, 1, mode=P.MODE_INT8)
    ms = _graph_ms(P, torch, [cap.graph]) / len(copies)
    nbytes = n * (k // 256 * 66) + 4 * (k + n)
    gbs = nbytes / ms / 1e6
    recs = [{"workload": "TQ2_0 (PTQTP plane) GEMV 8192x8192 batch 1 (30 rotated weight copies, graph replay)", "metric": "quant GEMV HBM GB/s",
             "value": round(gbs, 1), "unit": "GB/s", "us_per_launch": round(ms * 1e3, 3), "bytes_per_launch": nbytes,
             "roofline": {"bound": "hbm", "achieved": round(gbs, 1), "peak": peak, "unit": "GB/s", "frac": round(gbs / peak, 4),
                          "peak_source": src, "kernel": "decode_rows_kernel<TQ2_0, MB=1, fused act-quant>"}}]
    m = 256
    a = torch.randn((m, k), generator=g, device="cuda")
    c = torch.empty((m, n), device="cuda")
    torch.cuda.synchronize()
    fn = lambda: P.gemm_quant_nt_dev(copies[0], a, c, m, mode=P.MODE_AUTO)  # noqa: E731
    one = _timed(P, torch, fn, 5, 3)
    ms = _timed(P, torch, fn, max(5, min(5000, int(150.0 / one))), 0)
    tf = 2.0 * m * n * k / ms / 1e9
    recs.append({"workload": "TQ2_0 (PTQTP plane) GEMM 256x8192x8192 (bf16 tcgen05; the f32->bf16 activation pass is inside the timed call)",
                 "metric": "ternary GEMM TFLOPS", "value": round(tf, 1), "unit": "TFLOP/s", "ms": round(ms, 4),
                 "roofline": {"bound": "tensor", "achieved": round(tf, 1), "peak": burst, "unit": "TFLOP/s", "frac": round(tf / burst, 4),
                              "peak_source": tsrc + " (burst)", "kernel": "gemm_tc_kernel<TQ2_0, TN=256>"}})
    if want_cpu:
        xh = x.cpu().numpy()
        cores = oracle.set_threads(0)
        mm, arm = (lambda act: oracle.matmul_fast(F.TQ2_0, host, act)), ("AVX2 block dots" if oracle.has_simd(F.TQ2_0) else "scalar")
        pk = oracle.PackedRows.pack(F.TQ2_0, host, k)  # the reference's four-row pack (BlockTQ2_0x4), kept if it is the faster arm here
        if pk is not None and _cpu_time(lambda: pk.matmul(xh), 0.2, 50)[0] < _cpu_time(lambda: mm(xh), 0.2, 50)[0]:
            mm, arm = (lambda act: pk.matmul(act)), "AVX2 four-row packs (BlockTQ2_0x4)"
        sec, calls = _cpu_time(lambda: mm(xh), 1.5)
        oracle.set_threads(1)
        sec1, _ = _cpu_time(lambda: mm(xh), 1.0)
        oracle.set_threads(0)
        recs[0]["cpu_baseline"] = {"value": round(nbytes / sec / 1e9, 2), "unit": "GB/s", "cores": cores, "kind": "port",
                                   "sample": f"{calls} products, {sec * calls:.1f} s, " + arm,
                                   "single_thread": {"value": round(nbytes / sec1 / 1e9, 2), "unit": "GB/s"}}
        ah = a[:32].cpu().numpy()
        sec, calls = _cpu_time(lambda: mm(ah), 1.5)
        recs[1]["cpu_baseline"] = {"value": round(2.0 * 32 * n * k / sec / 1e12, 4), "unit": "TFLOP/s", "cores": cores, "kind": "port",
                                   "sample": f"32 of the 256 activation rows x the whole matrix, {calls} passes, {sec * calls:.1f} s, " + arm}
    return recs


def sub_multi(args, P, torch, rank: int, world: int, local: int) -> list[dict]:
    """The two exchange forms of the path over `world` GPUs (NVLink): the expert-parallel Q5_K MoE layer (128 / world
    experts per GPU) and the column-sharded Q4_K prefill with an all-gather of the output columns. Every rank
    also times the whole layer alone on its own GPU, so the speed-up is taken inside one run."""
    import torch.distributed as dist

    from fucina_b200 import formats as F
    from fucina_b200 import parallel as par

    ext = torch.cuda.ExternalStream(P.stream_ptr())
    h, f, E, topk = MOE["hidden"], MOE["ffn"], MOE["experts"], MOE["top_k"]
    recs = []

    def timed(fn, target_ms: float = 150.0) -> float:
        for _ in range(3):
            fn()
        P.synchronize()
        torch.cuda.synchronize()

        def run(steps):
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

        one = run(5)
        return run(max(5, min(2000, int(target_ms / max(one, 1e-3)))))

    # ---- the whole layer on one GPU (every rank, independently): the N = 1 figure of this very run ----
    full = _moe_stacks(P, torch, E, 1300)
    single_ms, _ = _moe_layer_ms(P, torch, full, 1024, 2, 3000 + 1024)
    single_ms = max_over_ranks(single_ms, world)
    single_tps = 1024 / single_ms * 1e3
    del full
    torch.cuda.empty_cache()

    per = E // world
    gate, up, down = _moe_stacks(P, torch, per, 1300 + 10 * rank)
    # the library's own exchange: NCCL communicator + peer-mapped arenas sized for the worst-case routing of the
    # largest case (every pair of every rank on one GPU)
    pairs_max = 1024 * topk
    fused = False
    try:
        P.tp_init_torch(dist, arena_bytes=(1 << 20) + pairs_max * h * 4 + world * pairs_max * (h * 2 + 8))
        fused = P.tp_peer_access()
    except Exception as e:  # noqa: BLE001
        recs.append({"workload": "fq_tp_init", "error": str(e)[:300]})

    def partial_rows(x_all, sel_all, w_all):
        o = torch.empty_like(x_all)
        P.moe_layer_ep_dev(gate, up, down, x_all, x_all.shape[0], topk, sel_all, w_all, rank * per, o)
        return o

    moe = par.ExpertParallelMoE(E, topk, lambda rows, le: rows)
    for T_total, scaling in ((1024 * world, "weak"), (1024, "strong")):
        T = T_total // world
        g = torch.Generator(device="cuda").manual_seed(3000 + 10 * rank + T_total)
        x = torch.randn((T, h), generator=g, device="cuda")
        logits = torch.randn((T, E), generator=g, device="cuda")
        sel = torch.empty((T, topk), dtype=torch.int32, device="cuda")
        wts = torch.empty((T, topk), device="cuda")
        out = torch.empty((T, h), device="cuda")
        torch.cuda.synchronize()
        forms = []
        if fused:
            def step_fused():
                P.router_topk_dev(logits, T, E, topk, True, sel, wts)
                P.moe_layer_ep(gate, up, down, x, T, topk, sel, wts, out, flags=P.EP_FUSED)

            forms.append(("fq_moe_layer_ep, fused form: token rows and result rows stored straight into peer memory over NVLink, "
                          "bounded flag waits", step_fused))

        def step_lib_nccl():
            P.router_topk_dev(logits, T, E, topk, True, sel, wts)
            P.moe_layer_ep(gate, up, down, x, T, topk, sel, wts, out, flags=P.EP_NCCL)

        forms.append(("fq_moe_layer_ep, baseline form: NCCL all-gather + reduce-scatter inside the library", step_lib_nccl))

        def step_nccl():
            with torch.cuda.stream(ext):
                P.router_topk_dev(logits, T, E, topk, True, sel, wts)
                moe.forward_gathered(x, sel, wts, partial_rows, exchange_dtype=torch.bfloat16 if T >= 512 else None)

        forms.append(("torch.distributed host logic: NCCL all-gather of token rows + reduce-scatter of partial sums", step_nccl))
        for name, fn in forms:
            try:
                ms = timed(fn)
                rec = {"workload": f"Q5_K MoE layer (hidden 2048, ffn 768, 128 experts, top-8), {T_total} tokens over {world} GPUs, {per} experts per GPU, {name}",
                       "metric": "MoE layer tok/s", "scaling": scaling, "n_gpus": world, "value": round(T_total / ms * 1e3, 1), "unit": "tok/s",
                       "ms": round(ms, 4), "single_gpu_1024_tokens": {"tok_per_s": round(single_tps, 1), "ms": round(single_ms, 4)},
                       "speedup_vs_single_gpu": round(T_total / ms * 1e3 / single_tps, 3)}
            except Exception as e:  # noqa: BLE001
                rec = {"workload": f"MoE expert-parallel, {name}", "error": str(e)[:300]}
            recs.append(rec)

    # ---- column-sharded prefill ----
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

        lin = par.ColumnShardedLinear(n, gemm)

        def step():
            with torch.cuda.stream(ext):
                lin.forward(a)

        try:
            if (hi - lo) * world == n:
                gathered = torch.empty((world, m, hi - lo), device="cuda")
                ms_lib = timed(lambda: P.gemm_quant_nt_tp(w, a, gathered, m, mode=P.MODE_TENSOR))
            else:
                ms_lib = None
            ms = timed(step)
            if ms_lib is not None and ms_lib < ms:
                ms = ms_lib
            ms_compute = timed(lambda: gemm(a))
            recs.append({"workload": f"Q4_K prefill {m}x{n}x{k}, output columns sharded over {world} GPUs, f32 all-gather (NCCL; "
                                     f"fq_gemm_quant_nt_tp {'%.4f ms' % ms_lib if ms_lib is not None else 'n/a'})",
                         "metric": "Q4_K prefill TFLOPS", "n_gpus": world, "value": round(2.0 * m * n * k / ms / 1e9, 1), "unit": "TFLOP/s",
                         "ms": round(ms, 4), "ms_compute_only": round(ms_compute, 4),
                         "gathered_MB_per_rank": round(m * n * 4 * (world - 1) / world / 1e6, 1)})
        except Exception as e:  # noqa: BLE001
            recs.append({"workload": f"column-sharded prefill {m}", "error": str(e)[:300]})
    barrier(world)
    try:
        P.tp_shutdown()
    except Exception:  # noqa: BLE001
        pass
    return recs


def _raw_blocks(P, torch, fmt: int, n: int, k: int, seed: int, n_mats: int = 1):
    """Seeded N(0, 0.02) rows through the library's device encoder, kept as raw GGUF blocks on the device (the layout
    the reference's kernels read)."""
    from fucina_b200 import formats as F

    g = torch.Generator(device="cuda").manual_seed(seed)
    rb = F.row_bytes(fmt, k)
    blocks = torch.empty(n_mats * n * rb, dtype=torch.uint8, device="cuda")
    for e in range(n_mats):
        w = torch.randn((n, k), generator=g, device="cuda", dtype=torch.float32) * 0.02
        torch.cuda.synchronize()
        P.quantize_rows_dev(fmt, w, n, k, blocks[e * n * rb:(e + 1) * n * rb])
        P.synchronize()
    return blocks


def sub_ref_kernels(args, P, torch, want_cpu: bool) -> list[dict]:
    """The reference's own CUDA kernels (its src/backend/cuda/kernels.cu, compiled unmodified for sm_100a by
    oracle/build.py into oracle/_ref) on this GPU and on the same shapes, launched with the grid shapes its host code
    uses: the recompiled-kernel baseline beside the records above. Device time only (CUDA events, graph replay where
    the record above uses one); the reference's host staging, PCIe copies and CPU phases are not in these figures."""
    from oracle import ref_cuda

    if not ref_cuda.available():
        return [{"workload": "reference CUDA kernels on this GPU", "unavailable": "oracle/_ref/libref_cuda.so was not built (no reference checkout at build time)"}]
    from fucina_b200 import formats as F

    st = P.stream_ptr()
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    impl = "reference kernels.cu compiled unmodified for sm_100a"
    recs = []
    g = torch.Generator(device="cuda").manual_seed(8000)
    k = 4096

    # decode stack, batch 1: four gemv launches per step, four rotated copies of the stack (473 MB > L2)
    rows = list(STACK_N)
    copies = [[_raw_blocks(P, torch, F.Q4_K, n, k, 8100 + 10 * c + i) for i, n in enumerate(rows)] for c in range(4)]
    x = torch.randn((1, k), generator=g, device="cuda")
    ys = [torch.empty((1, n), device="cuda") for n in rows]
    torch.cuda.synchronize()
    nb01 = F.row_bytes(F.Q4_K, k)
    with P.capture() as cap:
        for c in copies:
            for w, y, n in zip(c, ys, rows):
                ref_cuda.gemv(F.Q4_K, w.data_ptr(), x.data_ptr(), y.data_ptr(), k, n, 1, nb01, st)
    ms = _graph_ms(P, torch, [cap.graph]) / len(copies)
    recs.append({"workload": "Q4_K decode stack batch 1, reference gemv kernel (4 rotated stack copies, graph replay)", "impl": impl,
                 "kernel": "fucina_gemv_q4_K", "metric": "quant matmul HBM GB/s", "value": round(stack_bytes(1) / ms / 1e6, 1), "unit": "GB/s",
                 "us_per_step": round(ms * 1e3, 2)})
    del copies, cap
    torch.cuda.empty_cache()

    # Q8_0 GEMV 4096 x 4096
    n = 4096
    copies = [_raw_blocks(P, torch, F.Q8_0, n, k, 8200 + i) for i in range(30)]
    y = torch.empty((1, n), device="cuda")
    nb01 = F.row_bytes(F.Q8_0, k)
    torch.cuda.synchronize()
    with P.capture() as cap:
        for w in copies:
            ref_cuda.gemv(F.Q8_0, w.data_ptr(), x.data_ptr(), y.data_ptr(), k, n, 1, nb01, st)
    ms = _graph_ms(P, torch, [cap.graph]) / len(copies)
    nbytes = n * nb01 + 4 * k + 4 * n
    recs.append({"workload": "Q8_0 GEMV 4096x4096 batch 1, reference gemv kernel (30 rotated copies, graph replay)", "impl": impl,
                 "kernel": "fucina_gemv_q8_0", "metric": "quant GEMV HBM GB/s", "value": round(nbytes / ms / 1e6, 1), "unit": "GB/s",
                 "us_per_launch": round(ms * 1e3, 3)})
    del copies, cap
    torch.cuda.empty_cache()

    # Q4_K prefill 512 / 2048 x 14336 x 4096 on the reference's wmma tile kernel
    n = 14336
    w = _raw_blocks(P, torch, F.Q4_K, n, k, 8300)
    nb01 = F.row_bytes(F.Q4_K, k)
    for m in (512, 2048):
        a = torch.randn((m, k), generator=g, device="cuda")
        c = torch.empty((m, n), device="cuda")
        table = ref_cuda.dense_tiles(m)
        tiles = torch.tensor(table, dtype=torch.int32, device="cuda")
        n_tile, split_k = ref_cuda.plan(F.Q4_K, sms, len(table), n, k)
        part = torch.empty((split_k, m, n), device="cuda") if split_k > 1 else None
        torch.cuda.synchronize()
        fn = lambda: ref_cuda.mul_mm(F.Q4_K, w.data_ptr(), a.data_ptr(), tiles.data_ptr(), len(table), c.data_ptr(), k, n, nb01, nb01 * n,  # noqa: E731
                                     part.data_ptr() if part is not None else 0, split_k, m * n, n_tile, st)
        one = _timed(P, torch, fn, 3, 2)
        ms = _timed(P, torch, fn, max(3, min(500, int(150.0 / one))), 0)
        recs.append({"workload": f"Q4_K prefill GEMM {m}x{n}x{k}, reference tile kernel (wmma f16, N{n_tile} tiles, split-K {split_k})", "impl": impl,
                     "kernel": "fucina_mul_mm_mma_q4_K", "metric": "Q4_K prefill TFLOPS", "value": round(2.0 * m * n * k / ms / 1e9, 1), "unit": "TFLOP/s",
                     "ms": round(ms, 4)})
    del w
    torch.cuda.empty_cache()

    # the three grouped products of the Q5_K MoE layer at 1024 tokens (8192 routed rows over 128 experts)
    h, f, E, topk, T = MOE["hidden"], MOE["ffn"], MOE["experts"], MOE["top_k"], 1024
    gate = _raw_blocks(P, torch, F.Q5_K, f, h, 8400, E)
    up = _raw_blocks(P, torch, F.Q5_K, f, h, 8401, E)
    down = _raw_blocks(P, torch, F.Q5_K, h, f, 8402, E)
    sel = torch.topk(torch.randn((T, E), generator=g, device="cuda"), topk, dim=1).indices
    counts = torch.bincount(sel.reshape(-1), minlength=E).cpu().tolist()
    table = ref_cuda.grouped_tiles(counts)
    tiles = torch.tensor(table, dtype=torch.int32, device="cuda")
    pairs = T * topk
    xin = torch.randn((pairs, h), generator=g, device="cuda")
    gin = torch.randn((pairs, f), generator=g, device="cuda")
    og, ou, od = torch.empty((pairs, f), device="cuda"), torch.empty((pairs, f), device="cuda"), torch.empty((pairs, h), device="cuda")
    nb_h, nb_f = F.row_bytes(F.Q5_K, h), F.row_bytes(F.Q5_K, f)
    nt_gu, _ = ref_cuda.plan(F.Q5_K, sms, len(table), f, h, False)
    nt_d, _ = ref_cuda.plan(F.Q5_K, sms, len(table), h, f, False)
    torch.cuda.synchronize()

    def layer():
        ref_cuda.mul_mm(F.Q5_K, gate.data_ptr(), xin.data_ptr(), tiles.data_ptr(), len(table), og.data_ptr(), h, f, nb_h, nb_h * f, 0, 1, 0, nt_gu, st)
        ref_cuda.mul_mm(F.Q5_K, up.data_ptr(), xin.data_ptr(), tiles.data_ptr(), len(table), ou.data_ptr(), h, f, nb_h, nb_h * f, 0, 1, 0, nt_gu, st)
        ref_cuda.mul_mm(F.Q5_K, down.data_ptr(), gin.data_ptr(), tiles.data_ptr(), len(table), od.data_ptr(), f, h, nb_f, nb_f * h, 0, 1, 0, nt_d, st)

    one = _timed(P, torch, layer, 3, 2)
    ms = _timed(P, torch, layer, max(3, min(500, int(150.0 / one))), 0)
    recs.append({"workload": f"Q5_K MoE layer products at {T} tokens ({pairs} routed rows, {len(table)} tiles): gate, up and down grouped launches of the "
                             "reference tile kernel; its CPU gather / SwiGLU / scatter and PCIe round trips are not included", "impl": impl,
                 "kernel": "fucina_mul_mm_mma_q5_K", "metric": "MoE layer tok/s", "value": round(T / ms * 1e3, 1), "unit": "tok/s", "ms": round(ms, 4)})
    del gate, up, down, xin, gin, og, ou, od
    torch.cuda.empty_cache()

    # attention decode step at 8192 keys (the reference kernel gives one warp to a query row and head)
    H, KVH, D, KV = 32, 8, 128, 8192
    q = torch.randn((1, H, D), generator=g, device="cuda")
    kvs = [(torch.randn((KV, KVH, D), generator=g, device="cuda").to(torch.float16), torch.randn((KV, KVH, D), generator=g, device="cuda").to(torch.float16))
           for _ in range(6)]
    o = torch.empty((1, H, D), device="cuda")
    kvmap = torch.tensor([h * KVH // H for h in range(H)], dtype=torch.int32, device="cuda")
    torch.cuda.synchronize()
    with P.capture() as cap:
        for kk, vv in kvs:
            ref_cuda.attn_fwd(True, q.data_ptr(), kk.data_ptr(), vv.data_ptr(), o.data_ptr(), 0, kvmap.data_ptr(), 1, KV, H, KVH, D, KV - 1,
                              D ** -0.5, 0, True, st)
    ms = _graph_ms(P, torch, [cap.graph]) / len(kvs)
    nbytes = 2 * KV * KVH * D * 2
    recs.append({"workload": f"attention decode step, 1 query row, {H} heads / {KVH} kv heads, d {D}, {KV} keys, f16 KV, reference kernel (6 rotated KV copies, graph replay)",
                 "impl": impl, "kernel": "fucina_attn_fwd_f16", "metric": "attention KV GB/s", "value": round(nbytes / ms / 1e6, 1), "unit": "GB/s",
                 "us_per_step": round(ms * 1e3, 2)})
    return recs


def sub_records(args, P, torch, rank: int, world: int, local: int, want_cpu: bool) -> list[dict]:
    recs: list[dict] = []
    if world > 1:
        try:
            recs = sub_multi(args, P, torch, rank, world, local)
        except Exception as e:  # noqa: BLE001 - the headline value must survive a failing side record
            recs = [{"workload": "multi-GPU exchange forms", "error": str(e)[:300]}]
        return recs
    for fn in (sub_q8_0, sub_q6_k, sub_prefill, sub_moe, sub_ternary, sub_attention, sub_ref_kernels):
        try:
            recs.extend(fn(args, P, torch, want_cpu))
        except Exception as e:  # noqa: BLE001
            recs.append({"workload": fn.__name__, "error": str(e)[:300]})
        P.synchronize()
        torch.cuda.empty_cache()
    return recs


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
    ap.add_argument("--workload", default="stack", choices=["stack", "profile", "profile_q8", "profile_tc", "profile_moe", "attention", "q8_0", "prefill", "moe", "ternary", "all",
                                                                "tp_prefill", "ep_moe", "multi"])
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline legs")
    ap.add_argument("--no-sub", action="store_true", help="skip the records of the other configurations")
    ap.add_argument("--tokens", type=int, default=1024, help="tokens of the profile_moe case")
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
    if args.workload == "attention":
        import torch

        from fucina_b200 import provider as P

        P.init(0)
        for rec in sub_attention(args, P, torch, not args.no_cpu):
            print(json.dumps(rec), flush=True)
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
