"""The grouped entry point that allocates nothing, against the ordinary one.

Some hosts of this library run with a fixed GPU-memory footprint (ginn programs built on
PreallocGpuDevice count every device byte) or call from places where the CUDA allocator must not
be entered.  `ginn_b200_grouped_static` serves them: same kernel, descriptors in a fixed array
inside the library.  This file is collected last so that a failure here cannot hide others.
"""
import numpy as np
import pytest
import torch

from ginn_b200 import binding as B
from oracle import oracle as orc
from ginn_b200.binding import GROUPED_DW, GROUPED_DX, GROUPED_FORWARD

pytestmark = pytest.mark.gpu


def level(rng, specs):
    out = []
    for m, k, nc in specs:
        W = B.from_host((rng.standard_normal((m, k)) * 0.1).astype(np.float32))
        bias = B.from_host(rng.standard_normal(m).astype(np.float32))
        xs = [B.from_host(rng.standard_normal(k).astype(np.float32)) for _ in range(nc)]
        dys = [B.from_host(rng.standard_normal(m).astype(np.float32)) for _ in range(nc)]
        out.append((W, bias, xs, dys))
    return out


def run(gpu, call, lv):
    """Forward, dX and dW of one level through `call`; returns every output as host arrays."""
    ys = [[torch.zeros(W.shape[0], device="cuda") for _ in xs] for W, _, xs, _ in lv]
    dxs = [[torch.ones(W.shape[1], device="cuda") for _ in xs] for W, _, xs, _ in lv]
    dws = [B.colmajor(*W.shape, torch.float32, fill=0.5) for W, _, _, _ in lv]
    dbs = [torch.full((W.shape[0],), 0.25, device="cuda") for W, _, _, _ in lv]
    call(GROUPED_FORWARD, [gpu.Group(w=W, x_cols=xs, y_cols=y, bias=b)
                           for (W, b, xs, _), y in zip(lv, ys)])
    call(GROUPED_DX, [gpu.Group(w=W, y_cols=dys, dx_cols=dx) for (W, _, _, dys), dx in zip(lv, dxs)])
    call(GROUPED_DW, [gpu.Group(w=W, x_cols=xs, y_cols=dys, dw=dw, dbias=db)
                      for (W, _, xs, dys), dw, db in zip(lv, dws, dbs)])
    torch.cuda.synchronize()
    host = lambda ts: [B.to_host(t) for t in ts]
    return [host(y) for y in ys], [host(d) for d in dxs], host(dws), host(dbs)


def test_static_entry_point_matches_allocating_one_twice_in_a_row(gpu):
    rng = np.random.default_rng(77)
    first = level(rng, [(1024, 384, 40), (96, 40, 7)])
    second = level(rng, [(200, 64, 130)])      # different shape: the array is reused, not stale
    for lv in (first, second):
        want = run(gpu, gpu.grouped, lv)
        got = run(gpu, gpu.grouped_static, lv)
        # Same tolerance as the parity tests: relative Frobenius error 1e-5 (partial sums of a
        # split contraction are added atomically, so two runs need not agree bit for bit).
        for w_part, g_part in zip(want, got):
            for w, g in zip(w_part, g_part):
                w, g = (np.stack(w, 1), np.stack(g, 1)) if isinstance(w, list) else (w, g)
                assert orc.rel_frobenius(g, w) <= 1e-5


def test_static_entry_point_refuses_oversized_levels(gpu):
    W = B.colmajor(8, 8, torch.float32, fill=0.0)
    x = torch.zeros(8, device="cuda")
    cols = [x] * 20000      # 2 tables x 8 bytes x 20000 columns > 256 KiB
    with pytest.raises(gpu.GinnB200Error) as err:
        gpu.grouped_static(GROUPED_FORWARD, [gpu.Group(w=W, x_cols=cols, y_cols=cols)])
    assert err.value.status == 1 and "limit" in str(err.value)
