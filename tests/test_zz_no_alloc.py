"""The grouped entry point that allocates nothing.

Some hosts of this library run with a fixed GPU-memory footprint (ginn programs built on
PreallocGpuDevice count every device byte) or call from places where the CUDA allocator must not
be entered.  `ginn_b200_grouped_static` serves them: same kernels, descriptors in a fixed array
inside the library.  Checked here: its results against the ordinary entry point and against the
fp64 oracle, on two calls in a row; that a process which only ever uses this entry point sees
no change in free device memory across calls; and its refusals.  This file is collected last
so that a failure here cannot hide others.
"""
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from ginn_b200 import binding as B
from oracle import oracle as orc
from ginn_b200.binding import GROUPED_DW, GROUPED_DX, GROUPED_FORWARD
from helpers import TOL

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def level(rng, specs, dt=np.float32):
    """Host and device copies of a level: per group W, bias, x columns, dy columns."""
    out = []
    for m, k, nc in specs:
        W = (rng.standard_normal((m, k)) * 0.1).astype(dt)
        bias = rng.standard_normal(m).astype(dt)
        xs = [rng.standard_normal(k).astype(dt) for _ in range(nc)]
        dys = [rng.standard_normal(m).astype(dt) for _ in range(nc)]
        dev = (B.from_host(W), B.from_host(bias), [B.from_host(x) for x in xs],
               [B.from_host(d) for d in dys])
        out.append(((W, bias, xs, dys), dev))
    return out


def run(gpu, call, lv, tdt=torch.float32):
    """Forward, dX and dW of one level through `call`; returns every output as host arrays.
    The gradient slots start from non-zero values: every gradient write is `+=`."""
    devs = [d for _, d in lv]
    ys = [[torch.zeros(W.shape[0], device="cuda", dtype=tdt) for _ in xs] for W, _, xs, _ in devs]
    dxs = [[torch.ones(W.shape[1], device="cuda", dtype=tdt) for _ in xs] for W, _, xs, _ in devs]
    dws = [B.colmajor(*W.shape, tdt, fill=0.5) for W, _, _, _ in devs]
    dbs = [torch.full((W.shape[0],), 0.25, device="cuda", dtype=tdt) for W, _, _, _ in devs]
    call(GROUPED_FORWARD, [gpu.Group(w=W, x_cols=xs, y_cols=y, bias=b)
                           for (W, b, xs, _), y in zip(devs, ys)])
    call(GROUPED_DX, [gpu.Group(w=W, y_cols=dys, dx_cols=dx) for (W, _, _, dys), dx in zip(devs, dxs)])
    call(GROUPED_DW, [gpu.Group(w=W, x_cols=xs, y_cols=dys, dw=dw, dbias=db)
                      for (W, _, xs, dys), dw, db in zip(devs, dws, dbs)])
    torch.cuda.synchronize()
    stack = lambda ts: np.stack([B.to_host(t) for t in ts], 1)
    return [stack(y) for y in ys], [stack(d) for d in dxs], [B.to_host(t) for t in dws], \
        [B.to_host(t) for t in dbs]


def oracle_level(lv, dt):
    """The same four results from the fp64 restatement (ginn/autobatch.h:149-183 semantics:
    per group one product over the concatenated columns, bias broadcast, `+=` gradients)."""
    ys, dxs, dws, dbs = [], [], [], []
    for (W, bias, xs, dys), _ in lv:
        X, DY = np.stack(xs, 1), np.stack(dys, 1)
        W64, X64, DY64 = W.astype(np.float64), X.astype(np.float64), DY.astype(np.float64)
        ys.append((W64 @ X64 + bias.astype(np.float64)[:, None]).astype(dt))
        dxs.append((1.0 + W64.T @ DY64).astype(dt))
        dws.append((0.5 + DY64 @ X64.T).astype(dt))
        dbs.append((0.25 + DY64.sum(1)).astype(dt))
    return ys, dxs, dws, dbs


@pytest.mark.parametrize("dt", [np.float32, np.float16])
def test_static_entry_point_matches_allocating_one_and_oracle_twice_in_a_row(gpu, dt):
    rng = np.random.default_rng(77)
    tdt = torch.float32 if dt == np.float32 else torch.float16
    first = level(rng, [(1024, 384, 40), (96, 40, 7)], dt)
    second = level(rng, [(200, 64, 130)], dt)   # different shape: the array is reused, not stale
    tol = TOL[np.dtype(dt)]
    for lv in (first, second):
        want = run(gpu, gpu.grouped, lv, tdt)
        got = run(gpu, gpu.grouped_static, lv, tdt)
        ref = oracle_level(lv, dt)
        # Same tolerance as the parity tests (partial sums of a split contraction are added
        # atomically, so two runs need not agree bit for bit).
        for w_part, g_part, r_part in zip(want, got, ref):
            for w, g, r in zip(w_part, g_part, r_part):
                assert orc.rel_frobenius(g, w) <= tol
                assert orc.rel_frobenius(g, r) <= tol
    assert gpu.grouped_static_status(0, True) == 0


_CHILD = r"""
import sys
sys.path.insert(0, sys.argv[1])
import numpy as np, torch
from ginn_b200 import binding as B
torch.cuda.set_device(0)
rng = np.random.default_rng(5)
W = B.from_host((rng.standard_normal((256, 96)) * 0.1).astype(np.float32))
xs = [B.from_host(rng.standard_normal(96).astype(np.float32)) for _ in range(50)]
ys = [torch.zeros(256, device="cuda") for _ in range(50)]
dxs = [torch.zeros(96, device="cuda") for _ in range(50)]
dW = B.colmajor(256, 96, torch.float32, fill=0.0)
def calls():
    B.grouped_static(B.GROUPED_FORWARD, [B.Group(w=W, x_cols=xs, y_cols=ys)])
    B.grouped_static(B.GROUPED_DX, [B.Group(w=W, y_cols=ys, dx_cols=dxs)])
    B.grouped_static(B.GROUPED_DW, [B.Group(w=W, x_cols=xs, y_cols=ys, dw=dW)])
    torch.cuda.synchronize()
calls()                      # first use: symbol lookup, kernel image load
free0 = torch.cuda.mem_get_info(0)[0]
for _ in range(3):
    calls()
free1 = torch.cuda.mem_get_info(0)[0]
assert B.grouped_static_status(0, True) == 0
ref = B.to_host(W).astype(np.float64) @ np.stack([B.to_host(x) for x in xs], 1).astype(np.float64)
got = np.stack([B.to_host(y) for y in ys], 1)
err = float(np.linalg.norm(got - ref) / np.linalg.norm(ref))
print("FREE", free0, free1, "ERR", err)
sys.exit(0 if (free0 == free1 and err <= 1e-5) else 3)
"""


def test_static_entry_point_leaves_free_device_memory_unchanged():
    """A fresh process that uses no other entry point of the library: after the first call,
    further calls must not change the device's free memory (cudaMemGetInfo)."""
    res = subprocess.run([sys.executable, "-c", _CHILD, ROOT], capture_output=True, text=True,
                         timeout=600)
    print(res.stdout, res.stderr)
    assert res.returncode == 0, res.stdout + res.stderr


def test_static_entry_point_refuses_oversized_levels(gpu):
    W = B.colmajor(8, 8, torch.float32, fill=0.0)
    x = torch.zeros(8, device="cuda")
    cols = [x] * 20000      # 2 tables x 8 bytes x 20000 columns > 256 KiB
    with pytest.raises(gpu.GinnB200Error) as err:
        gpu.grouped_static(GROUPED_FORWARD, [gpu.Group(w=W, x_cols=cols, y_cols=cols)])
    assert err.value.status == 1 and "limit" in str(err.value)


def test_static_entry_point_refuses_a_capturing_stream(gpu):
    """Its descriptors come from a host buffer the next call overwrites, so recording the call
    into a CUDA graph would replay stale descriptors; the call says so instead."""
    W = B.colmajor(64, 32, torch.float32, fill=0.0)
    xs = [torch.zeros(32, device="cuda") for _ in range(4)]
    ys = [torch.zeros(64, device="cuda") for _ in range(4)]
    grp = [gpu.Group(w=W, x_cols=xs, y_cols=ys)]
    gpu.grouped_static(GROUPED_FORWARD, grp)          # first call outside any capture
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    status = None
    with torch.cuda.graph(g):
        try:
            gpu.grouped_static(GROUPED_FORWARD, grp)
        except gpu.GinnB200Error as e:
            status = e.status
    assert status == 2
