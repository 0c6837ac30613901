#!/usr/bin/env python
"""Benchmark of the Prod fwd+bwd hot path (large dense ProdNode, Half) on 1..N B200s.

One step = what ProdNode does for one forward + backward pass (ginn/node/prod.h:28-66) with the
gradients zeroed first, as Graph::reset_grad does (ginn/node.h:261-264):
    dA = 0; dB = 0;  C = A*B;  dA += dC*B^T;  dB += A^T*dC
A, B, dC are 8192 x 8192 fp16 (~N(0,1)), fp32 accumulation, column-major.

Multi-GPU (weak scaling): every rank owns an 8192-column shard of B, C and dC and a replica of A
(global B is 8192 x 8192*N).  Forward and dB need no exchange; dA is a sum over the sharded
columns, so the dA contributions are all-reduced (NCCL) on a side stream while the dB product
runs.

Prints ONE JSON line (rank 0).  `--impl reference` instead times the CPU restatement of the
reference's Eigen path (oracle/cpu_path.c) on the host cores, on a bounded sample.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# dram__bytes_read.sum + dram__bytes_write.sum of one hgemm_pair_kernel launch at 8192^3, from the
# ncu capture summarised in profiles/hgemm_pair_prod8192.md (mean of the three captured launches).
NCU_TRAFFIC_BYTES = {8192: 1.551e9}

METRIC = "prod_fwd_bwd_tflops"
UNIT = "TFLOP/s"
SIZE = 8192


def measured_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return json.load(f), "measured"
    except Exception:
        return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "20", "-i", str(self.gpu)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                smax.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(smax) if smax else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# ------------------------------------------------------------------------------------------
# CPU arm: the restated reference path on the host cores
# ------------------------------------------------------------------------------------------
def cpu_fwd_bwd(size: int, threads: int, steps: int, warmup: int):
    """Times `steps` fwd+bwd passes of the CPU port at size^3, fp16 storage.  Returns
    (TFLOP/s, seconds per step)."""
    from oracle import oracle as orc
    rng = np.random.default_rng(20244)
    a = np.asfortranarray(rng.standard_normal((size, size)).astype(np.float16))
    b = np.asfortranarray(rng.standard_normal((size, size)).astype(np.float16))
    dc = np.asfortranarray(rng.standard_normal((size, size)).astype(np.float16))
    L = orc.cpu_path()
    c = np.zeros((size, size), np.float16, order="F")
    da = np.zeros((size, size), np.float16, order="F")
    db = np.zeros((size, size), np.float16, order="F")

    def step():
        da.fill(0)
        db.fill(0)
        L.cpu_gemm(1, 0, 0, size, size, size, a.ctypes.data, size, b.ctypes.data, size,
                   c.ctypes.data, size, 0, threads)
        L.cpu_gemm(1, 0, 1, size, size, size, dc.ctypes.data, size, b.ctypes.data, size,
                   da.ctypes.data, size, 1, threads)
        L.cpu_gemm(1, 1, 0, size, size, size, a.ctypes.data, size, dc.ctypes.data, size,
                   db.ctypes.data, size, 1, threads)

    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = (time.perf_counter() - t0) / steps
    return 3 * 2 * size ** 3 / dt / 1e12, dt


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import oracle as orc
    threads = orc.cpu_path().cpu_max_threads()
    threads = max(threads, os.cpu_count() or 1)
    size = args.cpu_size
    val, dt = cpu_fwd_bwd(size, threads, max(args.steps, 1), min(args.warmup, 1))
    sample = (f"{size}^3 fp16 fwd+bwd (3 GEMMs) per step instead of {SIZE}^3; same operation "
              f"sequence, CPU port of the Eigen path (oracle/cpu_path.c), {threads} threads")
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16",
        "data": "synthetic",
        "config": {"workload": "C4 large dense ProdNode Half fwd+bwd 8192^3 (bounded CPU sample)",
                   "sample_size": size},
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": sample},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------
def run_gpu(args):
    import torch
    import torch.distributed as dist
    import ginn_b200 as gb
    from ginn_b200 import binding as B
    from ginn_b200.parallel import ShardedProd

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    n = args.size
    g = torch.Generator(device=dev)
    g.manual_seed(20244 + rank)
    ga = torch.Generator(device=dev)
    ga.manual_seed(20244)  # A is replicated: same seed on every rank

    def randn_cm(gen):  # column-major n x n fp16
        return torch.randn(n, n, device=dev, dtype=torch.float32, generator=gen).half().T

    A, Bm, dC = randn_cm(ga), randn_cm(g), randn_cm(g)
    Cm = torch.empty(n, n, device=dev, dtype=torch.float16).T
    dA = torch.empty(n, n, device=dev, dtype=torch.float16).T
    dB = torch.empty(n, n, device=dev, dtype=torch.float16).T
    comm_stream = torch.cuda.Stream(device=dev) if world > 1 else None
    main = torch.cuda.current_stream(dev)
    gemm_events = []

    def allreduce_async(t):
        if world == 1:
            return lambda: None
        ready = torch.cuda.Event()
        ready.record(main)
        comm_stream.wait_event(ready)
        with torch.cuda.stream(comm_stream):
            dist.all_reduce(t.T)  # contiguous storage of the column-major matrix
        return lambda: main.wait_stream(comm_stream)

    margin = args.sm_margin if args.sm_margin >= 0 else (8 if world > 1 else 0)
    gb.set_option("sm_margin", margin)
    prod = ShardedProd(lambda a, b, c, ta, tb, acc: gb.gemm(a, b, c, ta, tb, acc),
                       lambda t: t.zero_(), allreduce_async)

    def step(record=False):
        if not record:
            prod.step(A, Bm, dC, Cm, dA, dB)
            return
        # CUDA events around each of the three products, on the stream they are launched on
        evs = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
        state = {"first": True}

        def gemm_timed(a, b, c, ta, tb, acc):
            if state["first"]:
                evs[0].record()
                state["first"] = False
            gb.gemm(a, b, c, ta, tb, acc)

        timed = ShardedProd(gemm_timed, lambda t: t.zero_(), allreduce_async)
        timed.step(A, Bm, dC, Cm, dA, dB, between=lambda i: evs[i + 1].record())
        gemm_events.append(evs)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    status = gb.device_status(local, True)
    if status != 0:
        raise RuntimeError(f"device status {status:#x} after warm-up")

    sampler = ClockSampler(local) if rank == 0 else None
    if sampler:
        sampler.start()
    launches0 = gb.launch_count()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step(record=True)
    e1.record()
    barrier()
    launches = gb.launch_count() - launches0
    clocks = sampler.stop() if sampler else None
    ms = e0.elapsed_time(e1) / args.steps
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = t.item()
    kern_ms = []
    for evs in gemm_events:
        kern_ms += [evs[i].elapsed_time(evs[i + 1]) for i in range(3)]
    status = gb.device_status(local, True)
    if status != 0:
        raise RuntimeError(f"device status {status:#x} after the timed region")

    flops_step = 3 * 2 * n ** 3
    value = world * flops_step / (ms * 1e-3) / 1e12

    # ---- end to end through the C ABI with host buffers (pinned), copies inside the timed region
    e2e = None
    if not args.no_e2e:
        hA, hB, hdC = (torch.empty(n * n, dtype=torch.float16).pin_memory() for _ in range(3))
        hC, hdA, hdB = (torch.empty(n * n, dtype=torch.float16).pin_memory() for _ in range(3))
        hA.copy_(A.T.reshape(-1).cpu()); hB.copy_(Bm.T.reshape(-1).cpu()); hdC.copy_(dC.T.reshape(-1).cpu())

        # Copies run on their own streams so that they overlap the products inside a step:
        # dC arrives while C = A*B runs, C leaves while the two backward products run.
        h2d, d2h = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)

        def e2e_step():
            start = torch.cuda.Event()
            start.record(main)                      # previous step's products and copies are queued
            h2d.wait_event(start)
            d2h_prev = torch.cuda.Event()
            d2h_prev.record(d2h)
            main.wait_event(d2h_prev)               # results of the previous step have left
            ev_ab, ev_dc, ev_c = torch.cuda.Event(), torch.cuda.Event(), torch.cuda.Event()
            with torch.cuda.stream(h2d):
                A.T.reshape(-1).copy_(hA, non_blocking=True)
                Bm.T.reshape(-1).copy_(hB, non_blocking=True)
                ev_ab.record(h2d)
                dC.T.reshape(-1).copy_(hdC, non_blocking=True)
                ev_dc.record(h2d)
            main.wait_event(ev_ab)

            def after(i):
                if i == 0:
                    ev_c.record(main)
                    main.wait_event(ev_dc)
                    d2h.wait_event(ev_c)
                    with torch.cuda.stream(d2h):
                        hC.copy_(Cm.T.reshape(-1), non_blocking=True)

            prod.step(A, Bm, dC, Cm, dA, dB, between=after)
            done = torch.cuda.Event()
            done.record(main)
            d2h.wait_event(done)
            with torch.cuda.stream(d2h):
                hdA.copy_(dA.T.reshape(-1), non_blocking=True)
                hdB.copy_(dB.T.reshape(-1), non_blocking=True)

        def e2e_finish():
            main.wait_stream(d2h)
            main.wait_stream(h2d)

        e2e_step()
        e2e_finish()
        barrier()
        k = max(1, min(args.steps, 5))
        e0.record()
        for _ in range(k):
            e2e_step()
        e2e_finish()
        e1.record()
        barrier()
        ms_e = e0.elapsed_time(e1) / k
        if world > 1:
            t = torch.tensor([ms_e], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms_e = t.item()
        nbytes = 3 * n * n * 2
        e2e = {"value": world * flops_step / (ms_e * 1e-3) / 1e12, "unit": UNIT,
               "ms_per_step": ms_e, "h2d_bytes_per_step": nbytes, "d2h_bytes_per_step": nbytes}

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peaks, peak_src = measured_peaks()
    timed_s = ms * args.steps * 1e-3
    # Which measured cuBLAS figure is the fair denominator: the burst one for a short, cool run, the
    # sustained one when the board ran power-capped (clock well below maximum under sw_power_cap)
    # or the timed region is long.  Both fractions are reported.
    capped = bool(clocks and clocks.get("sm_mhz") and clocks.get("sm_max_mhz")
                  and "sw_power_cap" in clocks.get("reasons", [])
                  and clocks["sm_mhz"] < 0.8 * clocks["sm_max_mhz"])
    sustained = timed_s >= 1.0 or capped
    peak = peaks["bf16_tflops_sustained"] if sustained else peaks["bf16_tflops"]
    avg_kernel_ms = sum(kern_ms) / len(kern_ms)
    achieved = 2 * n ** 3 / (avg_kernel_ms * 1e-3) / 1e12
    roofline = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                "frac": achieved / peak, "traffic": NCU_TRAFFIC_BYTES.get(n),
                "frac_of_burst": achieved / peaks["bf16_tflops"],
                "frac_of_sustained": achieved / peaks["bf16_tflops_sustained"],
                "kernel": "hgemm_pair_kernel (tcgen05 cta_group::2; three transpose variants, "
                          "one launch each per step)",
                "avg_launch_ms": avg_kernel_ms,
                "peak_kind": f"{'sustained' if sustained else 'burst'} cuBLAS bf16, of {peak_src}"
                             + (" (board power-capped during the timed region)" if capped else "")}

    cpu_baseline = None
    if world == 1 and not args.no_cpu:
        from oracle import oracle as orc
        threads = max(orc.cpu_path().cpu_max_threads(), os.cpu_count() or 1)
        v, dt = cpu_fwd_bwd(args.cpu_size, threads, 1, 1)
        cpu_baseline = {"value": v, "unit": UNIT, "cores": threads, "kind": "port",
                        "sample": f"one fwd+bwd pass at {args.cpu_size}^3 fp16 ({dt:.2f} s), "
                                  f"CPU port of the Eigen path (oracle/cpu_path.c)"}

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": f"C4 large dense ProdNode Half fwd+bwd {n}^3 per GPU "
                               "(C=A*B, dA+=dC*B^T, dB+=A^T*dC, grads zeroed each step)",
                   "size": n, "l2": "inputs and outputs (768 MiB) exceed the 126 MB L2",
                   "sharding": "columns of B/C/dC per rank; dA all-reduced over NCCL" if world > 1
                   else "single GPU"},
        "clocks": clocks, "e2e": e2e, "gpu_launches": int(launches),
        "roofline": roofline, "cpu_baseline": cpu_baseline,
    }
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_affine(args):
    """Secondary workload (profiling aid): one fp32 AffineNode fwd+bwd, tanh, through the fused
    entry points.  Shapes default to config 5's hidden layer (1024 x 1024, batch 4096)."""
    import torch
    import ginn_b200 as gb
    from ginn_b200 import binding as B
    torch.cuda.set_device(0)
    m, n, k = args.m, args.n, args.k
    g = torch.Generator(device="cuda").manual_seed(20241)
    a = (6 / (0.5 * (m + k))) ** 0.5
    tdt = torch.float16 if args.dtype == "f16" else torch.float32
    W = ((torch.rand(k, m, device="cuda", generator=g) * 2 - 1) * a).to(tdt).T
    X = torch.randn(n, k, device="cuda", generator=g).to(tdt).T
    b = ((torch.rand(m, device="cuda", generator=g) * 2 - 1) * a).to(tdt)
    dY = torch.randn(n, m, device="cuda", generator=g).to(tdt).T
    Y = B.colmajor(m, n, tdt, fill=0.0)
    dW, dX = B.colmajor(m, k, tdt, fill=0.0), B.colmajor(k, n, tdt, fill=0.0)
    db = torch.zeros(m, device="cuda", dtype=tdt)

    def step():
        dW.zero_(); dX.zero_(); db.zero_()
        gb.affine_forward([gb.Pair(W, X)], b, gb.ACT_TANH, Y)
        gb.affine_backward([gb.PairGrad(W, X, dW, dX)], dY, Y, gb.ACT_TANH, db)

    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    assert gb.device_status(0, True) == 0
    print(json.dumps({"metric": "affine_fwd_bwd_tflops", "value": 3 * 2 * m * n * k / ms / 1e9,
                      "unit": UNIT, "n_gpus": 1, "steps": args.steps, "ms_per_step": ms,
                      "dtype": "f16" if args.dtype == "f16" else "f32 (3xTF32)", "data": "synthetic",
                      "config": {"workload": f"Affine tanh fwd+bwd W {m}x{k}, X {k}x{n}"}}),
          flush=True)


def run_step_ops(args):
    """The step's elementwise neighbours on sizes well beyond the 126 MB L2: Adam on 2^26 fp32
    parameters (32 algorithmic bytes per element: w, d, m, v read and written) and the picked
    negative log softmax on a 1024 x 65536 fp32 score matrix (forward 8 bytes per element:
    scores read, softmax written; backward 12: softmax read, gradient read and written).
    One JSON line with the three bandwidths against the measured copy bandwidth."""
    import torch
    import ginn_b200 as gb
    from ginn_b200 import binding as B

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    peaks, src = measured_peaks()
    n = 1 << 26
    w = torch.randn(n, device=dev)
    d = torch.randn(n, device=dev)
    m = torch.zeros(n, device=dev)
    v = torch.zeros(n, device=dev)
    rows, cols = 1024, 65536
    x = B.colmajor(rows, cols, torch.float32, dev)
    x.copy_(torch.randn(rows, cols, device=dev))
    smax = B.colmajor(rows, cols, torch.float32, dev, fill=0.0)
    dx = B.colmajor(rows, cols, torch.float32, dev, fill=0.0)
    idx = torch.randint(0, rows, (cols,), device=dev, dtype=torch.int32)
    val = torch.zeros(cols, device=dev)
    g = torch.ones(cols, device=dev)
    step = [0]

    def adam():
        step[0] += 1
        gb.adam_update(w, d, m, v, step[0])

    ops = {"adam": (adam, 32.0 * n),
           "pick_nll_forward": (lambda: gb.pick_nll_forward(x, idx, smax, val), 8.0 * rows * cols),
           "pick_nll_backward": (lambda: gb.pick_nll_backward(smax, idx, g, dx), 12.0 * rows * cols)}
    sampler = ClockSampler(0)
    sampler.start()
    out = {}
    launches0 = gb.launch_count()
    for name, (fn, nbytes) in ops.items():
        for _ in range(max(args.warmup, 3)):
            fn()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize(dev)
        e0.record()
        for _ in range(args.steps):
            fn()
        e1.record()
        torch.cuda.synchronize(dev)
        ms = e0.elapsed_time(e1) / args.steps
        gbs = nbytes / (ms * 1e-3) / 1e9
        out[name] = {"ms": ms, "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": gbs / peaks["hbm_gbs"], "bound": "hbm", "peak_source": src}
    clocks = sampler.stop()
    assert gb.device_status(0, True) == 0
    print(json.dumps({"metric": "step_ops_adam_gbs", "value": out["adam"]["achieved"], "unit": "GB/s",
                      "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 3),
                      "ms_per_step": out["adam"]["ms"], "higher_is_better": True, "scaling": "weak",
                      "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                      "config": {"workload": "Adam on 2^26 fp32 parameters; picked negative log softmax "
                                             "on 1024 x 65536 fp32 scores", "l2": "every array exceeds the 126 MB L2"},
                      "roofline": out["adam"], "ops": out, "clocks": clocks,
                      "gpu_launches": int(gb.launch_count() - launches0)}), flush=True)


def run_config_workload(args):
    """Secondary workloads: the other benchmark configurations (fp32), harnessed in
    ginn_b200/workloads.py.  Same timing rules as the main arm; one JSON line from rank 0."""
    import torch
    import torch.distributed as dist
    import ginn_b200 as gb
    from ginn_b200 import workloads as wl

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    extra = {}
    if args.workload == "attention_f32":
        w = wl.Attention(dev)
        metric, name = "attention_fwd_bwd_tflops", "C3 min-GPT attention via BatchedProd, fp32, 256 x (256x64x256)"
    elif args.workload == "lstm_flat":
        w = wl.LstmFlat(dev)
        extra["levels"], extra["nodes"] = 1, w.nodes
        metric, name = "autobatch_nodes_per_s", "C2 flat variant: one merged level, W 1024x384 on sum(len) gathered columns, fp32"
    elif args.workload == "lstm_autobatch":
        w = wl.LstmAutobatch(dev)
        t0 = time.perf_counter()
        w.rewrite()
        extra["rewrite_ms"] = (time.perf_counter() - t0) * 1e3
        extra["levels"], extra["nodes"] = w.T, w.nodes
        if args.cuda_graph:
            w.capture()
        extra["cuda_graph"] = bool(args.cuda_graph)
        metric, name = "autobatch_nodes_per_s", "C2 autobatched LSTM gates, fp32, 256 seqs len 5..40, W 1024x384"
    else:
        comm = torch.cuda.Stream(device=dev) if world > 1 else None

        def allreduce(t):
            """Sum over ranks on the communication stream; returns the wait for its result."""
            main = torch.cuda.current_stream(dev)
            ready = torch.cuda.Event()
            ready.record(main)
            comm.wait_event(ready)
            with torch.cuda.stream(comm):
                dist.all_reduce(t)
            return lambda: main.wait_stream(comm)
        w = wl.MlpDataParallel(dev, rank, world, allreduce=allreduce if world > 1 else None)
        metric, name = "mlp_dp_tflops", "C5 data-parallel MLP 784-1024-1024-10, fp32, batch 4096 per GPU, Adam"

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    for _ in range(max(args.warmup, 3)):
        w.step()
    barrier()
    assert gb.device_status(local, True) == 0
    sampler = ClockSampler(local) if rank == 0 else None
    if sampler:
        sampler.start()
    launches0 = gb.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    t0 = time.perf_counter()
    e0.record()
    for _ in range(args.steps):
        w.step()
    e1.record()
    barrier()
    wall_ms = (time.perf_counter() - t0) * 1e3 / args.steps
    ms = e0.elapsed_time(e1) / args.steps
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = t.item()
    clocks = sampler.stop() if sampler else None
    assert gb.device_status(local, True) == 0
    if rank == 0:
        tflops = world * w.flops / (ms * 1e-3) / 1e12
        per_unit = args.workload in ("lstm_autobatch", "lstm_flat")
        value = world * w.units / (ms * 1e-3) if per_unit else tflops
        line = {"metric": metric, "value": value,
                "unit": "nodes/s" if per_unit else UNIT,
                "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
                "ms_per_step": ms, "wall_ms_per_step": wall_ms, "tflops": tflops,
                "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                "dtype": "f32 (3xTF32)", "data": "synthetic", "config": {"workload": name},
                "clocks": clocks, "gpu_launches": int(gb.launch_count() - launches0)}
        line.update(extra)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--size", type=int, default=SIZE, help="matrix extent (default: the C4 config)")
    ap.add_argument("--cpu-size", type=int, default=3072, help="extent of the bounded CPU sample")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--sm-margin", type=int, default=-1,
                    help="SMs left free for NCCL while the dB product overlaps the all-reduce "
                         "(default: 0 on one GPU, 8 otherwise)")
    ap.add_argument("--workload", default="prod_f16", choices=["prod_f16", "affine_f32", "attention_f32", "lstm_autobatch", "lstm_flat", "mlp_dp", "step_ops"])
    ap.add_argument("--cuda-graph", action="store_true",
                    help="lstm_autobatch: replay the level sequence from a CUDA graph")
    ap.add_argument("--dtype", default="f32", choices=["f32", "f16"],
                    help="affine_f32 workload only: run the same Affine in Half instead")
    ap.add_argument("--m", type=int, default=1024)
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--k", type=int, default=1024)
    ap.add_argument("--force-path", type=int, default=0,
                    help="kernel choice override passed to the library (0 = automatic)")
    args = ap.parse_args()
    if args.force_path and args.impl != "reference":
        import ginn_b200
        ginn_b200.set_option("force_path", args.force_path)
    if args.impl == "reference":
        run_reference(args)
    elif args.workload == "affine_f32":
        run_affine(args)
    elif args.workload == "step_ops":
        run_step_ops(args)
    elif args.workload in ("attention_f32", "lstm_autobatch", "lstm_flat", "mlp_dp"):
        run_config_workload(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
