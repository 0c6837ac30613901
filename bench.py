#!/usr/bin/env python
"""Benchmark of ginn's dense-contraction hot path on 1..N B200s.

Headline workload (config 4): what ProdNode does for one forward + backward pass
(ginn/node/prod.h:28-66) with the gradients zeroed first, as Graph::reset_grad does
(ginn/node.h:261-264):
    dA = 0; dB = 0;  C = A*B;  dA += dC*B^T;  dB += A^T*dC
A, B, dC are 8192 x 8192 fp16 (~N(0,1)), fp32 accumulation, column-major.

Multi-GPU: ONE 8192^3 product, column-sharded (strong scaling).  Rank r owns columns
[r*8192/N, (r+1)*8192/N) of B, C and dC and a replica of A.  Forward and dB need no exchange; dA
is a sum over the sharded columns, so it is all-reduced (NCCL), panel by panel, while the later
panels and the dB product are computed.  The same line carries, under "secondary", the weak
variant (8192 columns per rank) and the data-parallel MLP of config 5, so that one record holds
all three scaling series.

On one GPU the line also carries "configs": the other benchmark configurations (Affine fp32,
autobatched LSTM gates, attention through BatchedProd, data-parallel MLP step), each with its own
timing, roofline fraction and CPU baseline.

Prints ONE JSON line (rank 0).  `--impl reference` instead times the CPU restatement of the
reference's Eigen path (oracle/cpu_path.c) on the host cores, on the same configuration.
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

METRIC = "prod_fwd_bwd_tflops"
UNIT = "TFLOP/s"
SIZE = 8192
PARITY_TOL_F16 = 5e-3   # relative Frobenius error against fp64, fp16 storage (the stated bound)


def measured_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return json.load(f), "measured"
    except Exception:
        return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


# C4: reset_grad of dA and dB on a second stream beside C = A*B (--fills-beside).  Measured: the
# step gains about 2 % (2.26 against 2.31 ms, three runs each) while the forward product, which
# then shares HBM with the fills, runs 1.5 % longer; off by default so that the per-launch times
# behind `roofline` are those of the products alone.
FILLS_BESIDE = False


def dram_traffic(kernel: str, size: int):
    """DRAM bytes per launch from the committed table of ncu captures (one entry per kernel and
    size, each with the command that produced it); None when the size was never captured."""
    try:
        with open(os.path.join(ROOT, "profiles", "dram_traffic.json")) as f:
            table = json.load(f)
        return table[kernel]["bytes_per_launch"].get(str(size))
    except Exception:
        return None


def c4_config(n: int, world: int) -> dict:
    """The configuration both arms are measured on (identical dictionaries)."""
    return {"workload": f"C4 large dense ProdNode Half fwd+bwd, one {n}^3 product "
                        "(C=A*B, dA+=dC*B^T, dB+=A^T*dC, grads zeroed each step)",
            "size": n, "gpus": world,
            "l2": "inputs and outputs (768 MiB) exceed the 126 MB L2",
            "sharding": (f"columns of B/C/dC split over {world} ranks; dA all-reduced over NCCL"
                         if world > 1 else "single GPU")}


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
def cpu_threads() -> int:
    from oracle import oracle as orc
    return max(orc.cpu_path().cpu_max_threads(), os.cpu_count() or 1)


class CpuMat:
    """Column-major host matrix for the C port (which takes pointers and leading dimensions)."""

    def __init__(self, rows, cols, dtype, rng=None, scale=1.0, lo=None):
        if rng is None:
            self.a = np.zeros((rows, cols), dtype, order="F")
        elif lo is not None:
            self.a = np.asfortranarray(rng.uniform(lo, -lo, (rows, cols)).astype(dtype))
        else:
            self.a = np.asfortranarray((rng.standard_normal((rows, cols)) * scale).astype(dtype))
        self.rows, self.cols = rows, cols

    @property
    def p(self):
        return self.a.ctypes.data


def cpu_gemm(L, dt, ta, tb, m, n, k, A, B, C, acc, threads, a_off=0, b_off=0, c_off=0):
    """C (+)= op(A) op(B) with the port; offsets are in elements (column blocks of a matrix)."""
    es = 4 if dt == 0 else 2
    L.cpu_gemm(dt, ta, tb, m, n, k, A.p + a_off * es, A.rows, B.p + b_off * es, B.rows,
               C.p + c_off * es, C.rows, acc, threads)


def timed(fn, steps, warmup):
    for _ in range(warmup):
        fn()
    t0 = time.perf_counter()
    for _ in range(steps):
        fn()
    return (time.perf_counter() - t0) / steps


def cpu_c4(size: int, threads: int, steps: int, warmup: int):
    """`steps` fwd+bwd passes of the CPU port at size^3, fp16 storage: (TFLOP/s, s per step)."""
    from oracle import oracle as orc
    L = orc.cpu_path()
    rng = np.random.default_rng(20244)
    a, b, dc = (CpuMat(size, size, np.float16, rng) for _ in range(3))
    c, da, db = (CpuMat(size, size, np.float16) for _ in range(3))

    def step():
        da.a.fill(0)
        db.a.fill(0)
        cpu_gemm(L, 1, 0, 0, size, size, size, a, b, c, 0, threads)
        cpu_gemm(L, 1, 0, 1, size, size, size, dc, b, da, 1, threads)
        cpu_gemm(L, 1, 1, 0, size, size, size, a, dc, db, 1, threads)

    dt = timed(step, steps, warmup)
    return 3 * 2 * size ** 3 / dt / 1e12, dt


def cpu_config_baselines(threads: int) -> dict:
    """The C port on the shapes of configs 1, 2 (recurrent and flat), 3 and 5, one to a few
    passes each (a few seconds in total).  Products only, as in the GPU flop counts."""
    from oracle import oracle as orc
    L = orc.cpu_path()
    rng = np.random.default_rng(20240)
    out = {}

    def affine_layer(m, k, n, need_dx=True):
        W, X, dY = CpuMat(m, k, np.float32, rng, 0.05), CpuMat(k, n, np.float32, rng), CpuMat(m, n, np.float32, rng)
        Y, dW, dX = CpuMat(m, n, np.float32), CpuMat(m, k, np.float32), CpuMat(k, n, np.float32)

        def run():
            cpu_gemm(L, 0, 0, 0, m, n, k, W, X, Y, 0, threads)
            cpu_gemm(L, 0, 0, 1, m, k, n, dY, X, dW, 1, threads)
            if need_dx:
                cpu_gemm(L, 0, 1, 0, k, n, m, W, dY, dX, 1, threads)
        return run

    # C1: one Affine 512 x 784 on 128 columns
    f = affine_layer(512, 784, 128)
    dt = timed(f, 20, 2)
    out["C1"] = {"value": 3 * 2 * 512 * 784 * 128 / dt / 1e12, "unit": UNIT, "ms_per_step": dt * 1e3,
                 "cores": threads, "kind": "port", "sample": "20 fwd+bwd passes, products only"}
    # C2: 40 levels of W 1024 x 384 on the live columns; flat: one level on all columns
    import torch
    lens = torch.randint(5, 41, (256,), generator=torch.Generator().manual_seed(20242)).numpy()
    live = [int((lens > t).sum()) for t in range(int(lens.max()))]   # the GPU harness's levels
    total = int(lens.sum())
    W = CpuMat(1024, 384, np.float32, rng, 0.05)
    X, dY = CpuMat(384, total, np.float32, rng), CpuMat(1024, total, np.float32, rng)
    Y, dX, dW = CpuMat(1024, total, np.float32), CpuMat(384, total, np.float32), CpuMat(1024, 384, np.float32)

    def levels():
        off = 0
        for n in live:
            cpu_gemm(L, 0, 0, 0, 1024, n, 384, W, X, Y, 0, threads, b_off=off * 384, c_off=off * 1024)
            cpu_gemm(L, 0, 1, 0, 384, n, 1024, W, dY, dX, 1, threads, b_off=off * 1024, c_off=off * 384)
            cpu_gemm(L, 0, 0, 1, 1024, 384, n, dY, X, dW, 1, threads, a_off=off * 1024, b_off=off * 384)
            off += n

    def flat():
        cpu_gemm(L, 0, 0, 0, 1024, total, 384, W, X, Y, 0, threads)
        cpu_gemm(L, 0, 1, 0, 384, total, 1024, W, dY, dX, 1, threads)
        cpu_gemm(L, 0, 0, 1, 1024, 384, total, dY, X, dW, 1, threads)

    for key, fn in (("C2", levels), ("C2_flat", flat)):
        dt = timed(fn, 2, 1)
        out[key] = {"value": total / dt, "unit": "nodes/s", "ms_per_step": dt * 1e3,
                    "tflops": 3 * 2 * 1024 * 384 * total / dt / 1e12, "cores": threads,
                    "kind": "port", "sample": "2 passes over the same level sizes, products only "
                                              "(no graph rewrite, no cell update)"}
    # C3: six batched products, 256 x (256 x 64 x 256)
    T, hs, nb = 256, 64, 256
    K_, Q, V, dO = (CpuMat(T, hs * nb, np.float32, rng, 0.35), CpuMat(hs, T * nb, np.float32, rng, 0.35),
                    CpuMat(hs, T * nb, np.float32, rng, 0.35), CpuMat(hs, T * nb, np.float32, rng))
    S, dS = CpuMat(T, T * nb, np.float32), CpuMat(T, T * nb, np.float32)
    O, dV, dQ, dK = (CpuMat(hs, T * nb, np.float32), CpuMat(hs, T * nb, np.float32),
                     CpuMat(hs, T * nb, np.float32), CpuMat(T, hs * nb, np.float32))

    def bg(ta, tb, m, n, k, A, B, C, acc):
        L.cpu_gemm_batched(0, ta, tb, m, n, k, A.p, A.rows, A.rows * (A.cols // nb), B.p, B.rows,
                           B.rows * (B.cols // nb), C.p, C.rows, C.rows * (C.cols // nb), nb, acc,
                           threads)

    def attention():
        bg(0, 0, T, T, hs, K_, Q, S, 0)
        bg(0, 0, hs, T, T, V, S, O, 0)
        bg(0, 1, hs, T, T, dO, S, dV, 1)
        bg(1, 0, T, T, hs, V, dO, dS, 1)
        bg(0, 1, T, hs, T, dS, Q, dK, 1)
        bg(1, 0, hs, T, T, K_, dS, dQ, 1)

    dt = timed(attention, 2, 1)
    out["C3"] = {"value": 6 * nb * 2 * T * hs * T / dt / 1e12, "unit": UNIT, "ms_per_step": dt * 1e3,
                 "cores": threads, "kind": "port",
                 "sample": "2 passes of the six batched products (softmax excluded, as in the flop count)"}
    # C5: the three layers of the MLP on 4096 columns
    layers = [affine_layer(1024, 784, 4096, False), affine_layer(1024, 1024, 4096),
              affine_layer(10, 1024, 4096)]

    def mlp():
        for f in layers:
            f()
    dt = timed(mlp, 2, 1)
    flops = 2 * sum(2 * a * b * 4096 for a, b in ((1024, 784), (1024, 1024), (10, 1024))) + \
        sum(2 * a * b * 4096 for a, b in ((1024, 1024), (10, 1024)))
    out["C5"] = {"value": flops / dt / 1e12, "unit": UNIT, "ms_per_step": dt * 1e3, "cores": threads,
                 "kind": "port", "sample": "2 passes of the eight products of a step (loss and Adam excluded)"}
    return out


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    world = int(os.environ.get("WORLD_SIZE", "1"))
    threads = cpu_threads()
    size = args.size
    steps, warmup = max(args.steps, 1), min(args.warmup, 1)
    val, dt = cpu_c4(size, threads, steps, warmup)
    single = None
    if not args.no_single_thread:
        # what the reference's own Makefile build does (no OpenMP): one thread, on a bounded
        # sample of the same operation sequence
        v1, dt1 = cpu_c4(args.cpu_size, 1, 1, 0)
        single = {"value": v1, "unit": UNIT, "cores": 1,
                  "sample": f"one fwd+bwd pass at {args.cpu_size}^3 ({dt1:.2f} s)"}
    sample = (f"{steps} fwd+bwd passes (3 GEMMs each) at the full {size}^3, CPU port of the Eigen "
              f"path (oracle/cpu_path.c, fp32 arithmetic on fp16 storage), {threads} threads")
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "strong" if world > 1 else "weak",
        "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": c4_config(size, world),
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": sample, "single_thread": single},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------
class Dist:
    """Rank bookkeeping and the collectives the harness needs (none on one GPU)."""

    def __init__(self):
        import torch
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(self.local)
        self.dev = torch.device("cuda", self.local)
        if self.world > 1:
            import torch.distributed as dist
            dist.init_process_group("nccl", device_id=self.dev)
        self.comm = torch.cuda.Stream(device=self.dev) if self.world > 1 else None

    def barrier(self):
        import torch
        if self.world > 1:
            import torch.distributed as dist
            dist.barrier()
        torch.cuda.synchronize(self.dev)

    def max_over_ranks(self, x: float) -> float:
        if self.world == 1:
            return x
        import torch
        import torch.distributed as dist
        t = torch.tensor([x], device=self.dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def sum_f64(self, t):
        if self.world > 1:
            import torch.distributed as dist
            dist.all_reduce(t)
        return t

    def allreduce_async(self, t):
        """Sum of a contiguous tensor over ranks on the communication stream; returns the
        function that makes the current stream wait for the result."""
        import torch
        import torch.distributed as dist
        main = torch.cuda.current_stream(self.dev)
        if self.world == 1:
            return lambda: None
        ready = torch.cuda.Event()
        ready.record(main)
        self.comm.wait_event(ready)
        with torch.cuda.stream(self.comm):
            dist.all_reduce(t)
        return lambda: main.wait_stream(self.comm)

    def close(self):
        if self.world > 1:
            import torch.distributed as dist
            dist.destroy_process_group()


class ProdShard:
    """Tensors and step of the sharded Prod pass on one rank: `ncols` columns of B, C, dC."""

    def __init__(self, D: Dist, n: int, first_col: int, ncols: int, panels: int, margin: int,
                 fills_beside: bool = None):
        import torch
        import ginn_b200 as gb
        from ginn_b200.parallel import ShardedProd
        self.D, self.n, self.first_col, self.ncols = D, n, first_col, ncols
        dev = D.dev
        ga = torch.Generator(device=dev).manual_seed(20244)       # A is replicated
        g = torch.Generator(device=dev).manual_seed(20245 + D.rank)

        def randn_cm(rows, cols, gen):  # column-major rows x cols fp16
            return torch.randn(cols, rows, device=dev, dtype=torch.float32, generator=gen).half().T

        self.A = randn_cm(n, n, ga)
        self.B, self.dC = randn_cm(n, ncols, g), randn_cm(n, ncols, g)
        empty = lambda cols: torch.empty(cols, n, device=dev, dtype=torch.float16).T
        self.C, self.dA, self.dB = empty(ncols), empty(n), empty(ncols)
        self.events = None

        def gemm(a, b, c, ta, tb, acc):
            if self.events is not None:
                ev = torch.cuda.Event(enable_timing=True)
                ev.record()
                self.events.append(ev)
            gb.gemm(a, b, c, ta, tb, acc)

        def overlapped(on):
            # SMs are kept free only for the products that run beside a reduction
            if D.world > 1 and margin > 0:
                gb.set_option("sm_margin", margin if on else 0)

        fill_stream = torch.cuda.Stream(device=dev)

        def zero_beside(ts):
            # reset_grad on a second stream: the fills (HBM-bound, no shared memory) run beside
            # the forward product, which does not touch the gradients
            main = torch.cuda.current_stream(dev)
            start = torch.cuda.Event()
            start.record(main)
            fill_stream.wait_event(start)
            with torch.cuda.stream(fill_stream):
                for t in ts:
                    t.zero_()
            return lambda: main.wait_stream(fill_stream)

        self.prod = ShardedProd(gemm, lambda t: t.zero_(),
                                lambda t: D.allreduce_async(t.T),  # contiguous storage of a panel
                                panels=panels if D.world > 1 else 1, overlapped=overlapped,
                                zero_beside=zero_beside if (FILLS_BESIDE if fills_beside is None
                                                            else fills_beside) else None)
        self.flops = 3 * 2 * n * n * ncols

    def step(self, between=None):
        self.prod.step(self.A, self.B, self.dC, self.C, self.dA, self.dB, between=between)

    def step_timed(self):
        """One step with a CUDA event before every product and one after the last; returns the
        events (durations are read after the timed region)."""
        import torch
        self.events = []
        after_gemms = torch.cuda.Event(enable_timing=True)
        self.step(between=lambda i: after_gemms.record() if i == 2 else None)
        end = torch.cuda.Event(enable_timing=True)
        end.record()                      # after the waits for the reductions
        evs, self.events = self.events + [after_gemms, end], None
        return evs

    def parity(self) -> dict:
        """Sampled entries of C, dB (local) and the reduced dA against an fp64 recomputation on
        the host from the very operands the GPU used (untimed).  Relative Frobenius error over
        each sampled block; the maximum over blocks and ranks is returned."""
        import torch
        D, n = self.D, self.n
        self.step()
        torch.cuda.synchronize(D.dev)
        rs = np.random.default_rng(99)                      # same samples on every rank
        rows = np.sort(rs.choice(n, 32, replace=False))
        gcols = np.sort(rs.choice(n, 64, replace=False))    # columns of dA = rows of B
        lcols = np.sort(rs.choice(self.ncols, min(64, self.ncols), replace=False))
        ti = lambda idx: torch.as_tensor(idx, device=D.dev)
        f64 = lambda t: t.double().cpu().numpy()
        A_rows, A_cols = f64(self.A[ti(rows)]), f64(self.A[:, ti(rows)])
        B_lc, dC_lc = f64(self.B[:, ti(lcols)]), f64(self.dC[:, ti(lcols)])
        errs = {}

        def rel(got, ref):
            return float(np.linalg.norm(got - ref) / max(np.linalg.norm(ref), 1e-300))

        errs["C"] = rel(f64(self.C[ti(rows)][:, ti(lcols)]), A_rows @ B_lc)
        errs["dB"] = rel(f64(self.dB[ti(rows)][:, ti(lcols)]), A_cols.T @ dC_lc)
        part = f64(self.dC[ti(rows)]) @ f64(self.B[ti(gcols)]).T   # this rank's share of dA
        ref = D.sum_f64(torch.as_tensor(part, device=D.dev)).cpu().numpy()
        errs["dA"] = rel(f64(self.dA[ti(rows)][:, ti(gcols)]), ref)
        worst = D.max_over_ranks(max(errs.values()))
        return {"checked": True, "max_rel": worst, "tol": PARITY_TOL_F16,
                "what": "32 x 64 sampled entries each of C, dB (per rank) and the all-reduced dA "
                        "against an fp64 host recomputation, relative Frobenius error, max over ranks",
                "rank0": errs, "ok": bool(worst <= PARITY_TOL_F16)}


def time_steps(D: Dist, step, steps: int, warmup: int):
    """Barrier + synchronize on both sides, CUDA events on the current stream, max over ranks."""
    import torch
    for _ in range(warmup):
        step()
    D.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    D.barrier()
    return D.max_over_ranks(e0.elapsed_time(e1) / steps)


def e2e_prod(D: Dist, P: ProdShard, steps: int):
    """The same pass through the C ABI with HOST buffers: every step copies this rank's operands
    in from pinned memory and its results out (C and dB shards, and this rank's slice of the
    reduced dA).  Three streams form a pipeline over two sets of device buffers: while step i
    computes, step i+1's operands arrive and step i-1's results leave, so a step costs what the
    slowest of the three takes (the host link, each way 0.4 GB per step on one GPU)."""
    import torch
    from ginn_b200.parallel import column_shard
    dev, n = D.dev, P.n
    main = torch.cuda.current_stream(dev)
    flat = lambda t: t.T.reshape(-1)
    pin = lambda t: torch.empty(t.numel(), dtype=torch.float16).pin_memory()
    hA, hB, hdC = pin(P.A), pin(P.B), pin(P.dC)
    hA.copy_(flat(P.A).cpu()); hB.copy_(flat(P.B).cpu()); hdC.copy_(flat(P.dC).cpu())
    s, c = column_shard(n, D.world, D.rank)
    sets = [P, ProdShard(D, n, P.first_col, P.ncols, P.prod.panels, 0)]
    sets[1].prod = P.prod  # same products, same reduction schedule
    hC, hdB, hdA = pin(P.C), pin(P.dB), pin(P.dA[:, s:s + c])
    h2d, d2h = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
    computed = [None, None]   # event: the products that read / wrote buffer set b are done
    drained = [None, None]    # event: the results of buffer set b have left the device

    def step(i):
        b = i & 1
        Q = sets[b]
        if computed[b] is not None:
            h2d.wait_event(computed[b])          # step i-2 no longer reads these operands
        arrived = torch.cuda.Event()
        with torch.cuda.stream(h2d):
            flat(Q.A).copy_(hA, non_blocking=True)
            flat(Q.B).copy_(hB, non_blocking=True)
            flat(Q.dC).copy_(hdC, non_blocking=True)
            arrived.record(h2d)
        main.wait_event(arrived)
        if drained[b] is not None:
            main.wait_event(drained[b])          # step i-2's results are out of these buffers
        Q.prod.step(Q.A, Q.B, Q.dC, Q.C, Q.dA, Q.dB)
        computed[b] = torch.cuda.Event()
        computed[b].record(main)
        d2h.wait_event(computed[b])
        with torch.cuda.stream(d2h):
            hC.copy_(flat(Q.C), non_blocking=True)
            hdA.copy_(flat(Q.dA[:, s:s + c]), non_blocking=True)
            hdB.copy_(flat(Q.dB), non_blocking=True)
            drained[b] = torch.cuda.Event()
            drained[b].record(d2h)

    def finish():
        main.wait_stream(d2h)
        main.wait_stream(h2d)

    for i in range(4):
        step(i)
    finish()
    D.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        step(i)
    finish()
    e1.record()
    D.barrier()
    ms = D.max_over_ranks(e0.elapsed_time(e1) / steps)
    h2d_b = 2 * (P.A.numel() + P.B.numel() + P.dC.numel())
    d2h_b = 2 * (P.C.numel() + P.dB.numel() + P.dA[:, s:s + c].numel())
    del sets
    return ms, h2d_b, d2h_b


def fp32_ceiling(peaks):
    """Ceiling of a 3xTF32 kernel in useful fp32 flops: the measured bf16 burst rate, halved for
    TF32 operands, divided by the three tensor-core products every term costs."""
    return peaks["bf16_tflops"] / 2.0 / 3.0


def run_mlp_dp(D: Dist, steps: int, warmup: int) -> dict:
    """Config 5 step (fwd, loss, bwd, bucketed all-reduce, Adam); replicas must stay identical."""
    import torch
    from ginn_b200 import workloads as wl
    w = wl.MlpDataParallel(D.dev, D.rank, D.world,
                           allreduce=D.allreduce_async if D.world > 1 else None)
    # the first all-reduces of a new size still set NCCL channels up: at least ten untimed steps
    # when ranks communicate (0.55 ms measured after three, 0.46-0.50 after ten, at N = 2)
    warm = max(warmup, 10 if D.world > 1 else 3)
    for _ in range(3):
        w.step()
    torch.cuda.synchronize(D.dev)
    # the kernel launches of a step replayed from two CUDA graphs (collectives and Adam stay
    # ordinary calls), the same at every N: with eight processes on one host the launches
    # otherwise take the host as long as the GPU
    try:
        w.capture()
        launched = "two CUDA graphs per step (before / after the first all-reduce); NCCL and Adam called directly"
    except Exception as e:
        launched = f"call by call (graph capture failed: {type(e).__name__})"
    ms = time_steps(D, w.step, max(steps, 30) if D.world > 1 else steps, warm)
    out = {"ms_per_step": ms, "warmup": warm, "tflops": D.world * w.flops / (ms * 1e-3) / 1e12,
           "flops_per_step_per_gpu": w.flops, "loss": float(w.loss), "launched": launched}
    if D.world > 1:
        import torch.distributed as dist
        ref = w.params.clone()
        dist.broadcast(ref, 0)
        out["replica_max_abs_diff"] = D.max_over_ranks(float((w.params - ref).abs().max()))
    return out


def run_cpp_autobatch() -> dict:
    """Config 2 through the C++ host layer (ginn_b200/include/ginn/autobatch.h): one graph node
    per sequence and step, tensors from a preallocated device, Autobatch(g) and the level
    preparation inside the timed region.  Runs tests/cpp/bench_autobatch (built on demand)."""
    cpp = os.path.join(ROOT, "tests", "cpp")
    exe = os.path.join(cpp, "bench_autobatch")
    try:
        subprocess.run(["make", "-C", cpp, "bench_autobatch"], check=True, capture_output=True,
                       timeout=300)
        res = subprocess.run([exe, "5", "20"], capture_output=True, text=True, timeout=300)
        line = [ln for ln in res.stdout.splitlines() if ln.startswith("{")][-1]
        out = json.loads(line)
        out["what"] = ("C++ BatchedGraph on per-node tensors: rewrite_ms = Autobatch(g); "
                       "first_pass = forward + reset_grad + backward with the one-time level "
                       "preparation; replay = the same pass on the prepared schedule, launch by "
                       "launch; graph = the pass replayed from a CUDA graph "
                       "(BatchedGraph::capture_pass); host clock around device synchronisation")
        return out
    except Exception as e:  # the headline does not depend on it
        return {"error": f"{type(e).__name__}: {e}"[:300]}


def run_configs(D: Dist, args, peaks) -> dict:
    """Configs 1, 2 (recurrent and flat), 3 and 5 on one GPU: ms per step, useful TFLOP/s or
    nodes/s, fraction of the 3xTF32 ceiling, and the CPU port on the same shapes."""
    import torch
    import ginn_b200 as gb
    from ginn_b200 import binding as B
    from ginn_b200 import workloads as wl
    dev = D.dev
    ceil = fp32_ceiling(peaks)
    steps, warmup = max(args.config_steps, 1), 3
    cpu = cpu_config_baselines(cpu_threads()) if not args.no_cpu else {}
    out = {}

    def entry(key, name, ms, flops, extra=None):
        tf = flops / (ms * 1e-3) / 1e12
        e = {"workload": name, "ms_per_step": ms, "tflops": tf, "dtype": "f32 (3xTF32)",
             "roofline": {"bound": "tensor", "achieved": tf, "peak": ceil, "unit": UNIT,
                          "frac": tf / ceil,
                          "peak_kind": "measured bf16 burst / 2 (TF32) / 3 (products per term)"},
             "cpu_baseline": cpu.get(key)}
        e.update(extra or {})
        out[key] = e

    # C1
    w = wl.AffineLayer(dev, 512, 128, 784)
    launches0 = gb.launch_count()
    ms_py = time_steps(D, w.step, steps, warmup)
    launches = (gb.launch_count() - launches0) // (steps + warmup)
    ms = time_steps(D, wl.graphed(w.step), 10 * steps, warmup)
    entry("C1", "Affine tanh fwd+bwd fp32: W 512x784, X 784x128", ms, w.flops,
          {"us_per_step": ms * 1e3, "us_per_step_launched_from_python": ms_py * 1e3,
           "launches_per_step": launches,
           "note": "replayed from a CUDA graph (device time); launched call by call from "
                   "Python the step is bound by the host"})
    # C2 recurrent: prepared levels replayed from a CUDA graph; the rewrite (host grouping +
    # descriptor upload) timed separately and added for the with-rewrite figure
    w = wl.LstmAutobatch(dev)
    t0 = time.perf_counter()
    w.rewrite()
    torch.cuda.synchronize(dev)
    rewrite_ms = (time.perf_counter() - t0) * 1e3
    ms_launch = time_steps(D, w.step, max(steps // 4, 2), 2)
    w.capture()
    ms = time_steps(D, w.step, steps, warmup)
    entry("C2", "autobatched LSTM gates fp32: 256 seqs len 5..40, W 1024x384, 40 dependent levels",
          ms, w.flops,
          {"nodes": w.nodes, "levels": w.T, "nodes_per_s": w.nodes / (ms * 1e-3),
           "nodes_per_s_launched_from_python": w.nodes / (ms_launch * 1e-3),
           "rewrite_ms": rewrite_ms,
           "nodes_per_s_with_rewrite": w.nodes / ((ms_launch + rewrite_ms) * 1e-3),
           "note": "replayed from a CUDA graph; with_rewrite = one rewrite + one pass launched "
                   "level by level, as a graph built anew for every batch needs"})
    del w
    out["C2"]["cpp_batched_graph"] = run_cpp_autobatch()
    # C2 flat
    w = wl.LstmFlat(dev)
    ms = time_steps(D, w.step, steps, warmup)
    entry("C2_flat", "C2 flat variant: one merged level, W 1024x384 on sum(len) gathered columns",
          ms, w.flops, {"nodes": w.nodes, "nodes_per_s": w.nodes / (ms * 1e-3)})
    del w
    # C3
    w = wl.Attention(dev)
    ms = time_steps(D, w.step, steps, warmup)
    entry("C3", "min-GPT attention via BatchedProd fp32: 256 x (256x64x256), fwd+bwd", ms, w.flops)
    del w
    # C5
    r = run_mlp_dp(D, steps, warmup)
    entry("C5", "data-parallel MLP 784-1024-1024-10 fp32, batch 4096 per GPU, softmax-CE, Adam",
          r["ms_per_step"], r["flops_per_step_per_gpu"], {"loss": r["loss"]})
    assert gb.device_status(D.local, True) == 0
    torch.cuda.empty_cache()
    return out


def run_gpu(args):
    import torch
    import ginn_b200 as gb
    from ginn_b200.parallel import column_shard

    D = Dist()
    world, rank = D.world, D.rank
    n = args.size
    margin = args.sm_margin if args.sm_margin >= 0 else (8 if world > 1 else 0)
    first, ncols = column_shard(n, world, rank)
    # a panel's product must be long enough to hide the reduction of the panel before it: with
    # 1024 columns per rank (N = 8) one panel measured 0.83 ms per step against 0.92 with two
    pick_panels = lambda cols: args.panels if args.panels > 0 else (2 if cols >= 2048 else 1)
    P = ProdShard(D, n, first, ncols, pick_panels(ncols), margin)
    warmup = max(args.warmup, 3)

    for _ in range(warmup):
        P.step()
    D.barrier()
    status = gb.device_status(D.local, True)
    if status != 0:
        raise RuntimeError(f"device status {status:#x} after warm-up")

    sampler = ClockSampler(D.local) if rank == 0 else None
    if sampler:
        sampler.start()
    launches0 = gb.launch_count()
    gemm_events = []
    D.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        gemm_events.append(P.step_timed())
    e1.record()
    D.barrier()
    launches = gb.launch_count() - launches0
    clocks = sampler.stop() if sampler else None
    ms = D.max_over_ranks(e0.elapsed_time(e1) / args.steps)
    gemm_ms = sum(evs[0].elapsed_time(evs[-2]) for evs in gemm_events) / len(gemm_events)
    launches_per_step = len(gemm_events[0]) - 2
    # mean duration of every product of a step, in launch order, and of the wait for the
    # reductions that is left after the last product
    breakdown = [sum(evs[i].elapsed_time(evs[i + 1]) for evs in gemm_events) / len(gemm_events)
                 for i in range(launches_per_step + 1)]
    status = gb.device_status(D.local, True)
    if status != 0:
        raise RuntimeError(f"device status {status:#x} after the timed region")

    total_flops = 3 * 2 * n ** 3                     # the whole job, however it is sharded
    value = total_flops / (ms * 1e-3) / 1e12
    flops_launches = P.flops                         # this rank's three products
    parity = P.parity()

    e2e = None
    if not args.no_e2e:
        ms_e, h2d_b, d2h_b = e2e_prod(D, P, args.steps)
        e2e = {"value": total_flops / (ms_e * 1e-3) / 1e12, "unit": UNIT, "ms_per_step": ms_e,
               "h2d_bytes_per_step": h2d_b, "d2h_bytes_per_step": d2h_b,
               "bytes_are": "per rank" if world > 1 else "total"}

    secondary = {}
    if world > 1 and not args.no_secondary:
        del P
        torch.cuda.empty_cache()
        Pw = ProdShard(D, n, rank * n, n, pick_panels(n), margin)  # weak: n columns per rank
        ms_w = time_steps(D, Pw.step, args.steps, warmup)
        secondary["c4_weak"] = {
            "scaling": "weak", "ms_per_step": ms_w, "value": world * Pw.flops / (ms_w * 1e-3) / 1e12,
            "unit": UNIT, "workload": f"{n}^3 per rank (global B is {n} x {n * world})",
            "parity": Pw.parity()}
        del Pw
        torch.cuda.empty_cache()
        r = run_mlp_dp(D, args.steps, warmup)
        secondary["c5_mlp_dp"] = {"scaling": "weak", "unit": UNIT, "value": r["tflops"], **r,
                                  "workload": "C5 data-parallel MLP, 4096 columns per rank, "
                                              "bucketed NCCL all-reduce overlapped with backward"}

    if rank != 0:
        D.close()
        return

    peaks, peak_src = measured_peaks()
    achieved = flops_launches / (gemm_ms * 1e-3) / 1e12
    peak = peaks["bf16_tflops"]
    roofline = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": UNIT,
                "frac": achieved / peak,
                "frac_of_sustained": achieved / peaks["bf16_tflops_sustained"],
                "traffic": dram_traffic("hgemm_pair_kernel", n) if world == 1 else None,
                "kernel": "hgemm_pair_kernel (tcgen05 cta_group::2; NN, NT, TN variants)",
                "launches_per_step": launches_per_step,
                "avg_launch_ms": gemm_ms / launches_per_step,
                "peak_kind": f"burst cuBLAS bf16, of {peak_src}; frac_of_sustained = against the "
                             "seconds-long power-capped figure"}

    cpu_baseline, configs = None, None
    if world == 1:
        if not args.no_cpu:
            threads = cpu_threads()
            v, dt = cpu_c4(args.cpu_size, threads, 1, 1)
            cpu_baseline = {"value": v, "unit": UNIT, "cores": threads, "kind": "port",
                            "sample": f"one fwd+bwd pass at {args.cpu_size}^3 fp16 ({dt:.2f} s), CPU "
                                      "port of the Eigen path (oracle/cpu_path.c); the reference "
                                      "arm times the full size"}
        if not args.no_configs:
            configs = run_configs(D, args, peaks)
            c5 = configs["C5"]
            secondary["c5_mlp_dp"] = {"scaling": "weak", "unit": UNIT, "value": c5["tflops"],
                                      "ms_per_step": c5["ms_per_step"], "tflops": c5["tflops"]}
            secondary["c4_weak"] = {"scaling": "weak", "ms_per_step": ms, "value": value, "unit": UNIT}

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "strong" if world > 1 else "weak", "vs_baseline": None, "dtype": "f16",
        "data": "synthetic", "config": c4_config(n, world),
        "clocks": clocks, "e2e": e2e, "gpu_launches": int(launches),
        "roofline": roofline, "cpu_baseline": cpu_baseline, "parity": parity,
        "secondary": secondary or None, "configs": configs,
        "dA_panels": pick_panels(ncols) if world > 1 else 1, "sm_margin_beside_collectives": margin,
        "step_breakdown_ms": {"products_in_launch_order": breakdown[:-1],
                              "exposed_wait_for_reductions": breakdown[-1]},
    }
    print(json.dumps(line), flush=True)
    D.close()
    if not parity["ok"] or any(not s.get("parity", {"ok": True})["ok"] for s in secondary.values()):
        sys.exit(4)


def run_affine(args):
    """Profiling aid: one AffineNode fwd+bwd, tanh, through the fused entry points.  Shapes
    default to config 5's hidden layer (1024 x 1024, batch 4096)."""
    import torch
    import ginn_b200 as gb
    from ginn_b200 import workloads as wl
    D = Dist()
    w = wl.AffineLayer(D.dev, args.m, args.n, args.k, half=args.dtype == "f16")
    step = wl.graphed(w.step) if args.cuda_graph else w.step
    ms = time_steps(D, step, args.steps, max(args.warmup, 3))
    assert gb.device_status(0, True) == 0
    print(json.dumps({"metric": "affine_fwd_bwd_tflops", "value": w.flops / ms / 1e9,
                      "unit": UNIT, "n_gpus": 1, "steps": args.steps, "ms_per_step": ms,
                      "dtype": "f16" if args.dtype == "f16" else "f32 (3xTF32)", "data": "synthetic",
                      "config": {"workload": f"Affine tanh fwd+bwd W {args.m}x{args.k}, X {args.k}x{args.n}"}}),
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
    """One of the other configurations alone (profiling aid; the default run reports them all in
    its "configs" block).  Same timing rules as the main arm; one JSON line from rank 0."""
    import torch
    import ginn_b200 as gb
    from ginn_b200 import workloads as wl

    D = Dist()
    dev, world, rank = D.dev, D.world, D.rank
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
        w = wl.MlpDataParallel(dev, rank, world, allreduce=D.allreduce_async if world > 1 else None)
        metric, name = "mlp_dp_tflops", "C5 data-parallel MLP 784-1024-1024-10, fp32, batch 4096 per GPU, Adam"

    for _ in range(max(args.warmup, 3)):
        w.step()
    D.barrier()
    assert gb.device_status(D.local, True) == 0
    sampler = ClockSampler(D.local) if rank == 0 else None
    if sampler:
        sampler.start()
    launches0 = gb.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    D.barrier()
    t0 = time.perf_counter()
    e0.record()
    for _ in range(args.steps):
        w.step()
    e1.record()
    D.barrier()
    wall_ms = (time.perf_counter() - t0) * 1e3 / args.steps
    ms = D.max_over_ranks(e0.elapsed_time(e1) / args.steps)
    clocks = sampler.stop() if sampler else None
    assert gb.device_status(D.local, True) == 0
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
    D.close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--size", type=int, default=SIZE, help="matrix extent (default: the C4 config)")
    ap.add_argument("--cpu-size", type=int, default=3072,
                    help="extent of the bounded CPU samples (cpu_baseline of the GPU arm, "
                         "single-thread figure of the reference arm)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-configs", action="store_true", help="skip the configs block (1 GPU)")
    ap.add_argument("--no-secondary", action="store_true",
                    help="N > 1: skip the weak-scaling and data-parallel MLP series")
    ap.add_argument("--no-single-thread", action="store_true",
                    help="reference arm: skip the single-thread sample")
    ap.add_argument("--config-steps", type=int, default=20, help="timed steps per configs entry")
    ap.add_argument("--panels", type=int, default=0,
                    help="column panels of dA, each all-reduced as soon as it is computed (N > 1); "
                         "0 = two while a rank holds at least 2048 columns, else one")
    ap.add_argument("--sm-margin", type=int, default=-1,
                    help="SMs left free for NCCL by the products that run beside a reduction "
                         "(default: 0 on one GPU, 8 otherwise)")
    ap.add_argument("--workload", default="prod_f16", choices=["prod_f16", "affine_f32", "attention_f32", "lstm_autobatch", "lstm_flat", "mlp_dp", "step_ops"])
    ap.add_argument("--cuda-graph", action="store_true",
                    help="lstm_autobatch, affine_f32: replay the step from a CUDA graph")
    ap.add_argument("--dtype", default="f32", choices=["f32", "f16"],
                    help="affine_f32 workload only: run the same Affine in Half instead")
    ap.add_argument("--m", type=int, default=1024)
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--k", type=int, default=1024)
    ap.add_argument("--force-path", type=int, default=0,
                    help="kernel choice override passed to the library (0 = automatic)")
    ap.add_argument("--pair-group-m", type=int, default=0,
                    help="rasterisation group of the CTA-pair kernel (0 = library default)")
    ap.add_argument("--pair-l2-hint", type=int, default=-1,
                    help="L2 eviction hints of the CTA-pair kernel, 0..3 (-1 = library default)")
    ap.add_argument("--fills-beside", action="store_true",
                    help="C4: clear dA and dB on a second stream beside the forward product")
    ap.add_argument("--pdl", type=int, default=1,
                    help="0: launch without programmatic dependent launch (A/B aid)")
    args = ap.parse_args()
    global FILLS_BESIDE
    FILLS_BESIDE = args.fills_beside
    if args.force_path and args.impl != "reference":
        import ginn_b200
        ginn_b200.set_option("force_path", args.force_path)
    if args.pair_group_m and args.impl != "reference":
        import ginn_b200
        ginn_b200.set_option("pair_group_m", args.pair_group_m)
    if args.pair_l2_hint >= 0 and args.impl != "reference":
        import ginn_b200
        ginn_b200.set_option("pair_l2_hint", args.pair_l2_hint)
    if not args.pdl and args.impl != "reference":
        import ginn_b200
        ginn_b200.set_option("pdl", 0)
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
