"""GPU parity of the grouped (autobatch level) entry point: one launch for all groups of a
level must equal the per-node products the un-batched graph computes (the before/after
protocol of test/autobatch.cpp:37-70)."""
import numpy as np
import pytest
import torch

from oracle import oracle as orc
from ginn_b200 import binding as B
from ginn_b200.binding import GROUPED_DW, GROUPED_DX, GROUPED_FORWARD
from helpers import check, check_elementwise, randn

pytestmark = pytest.mark.gpu


def make_level(rng, specs):
    """specs: list of (m, k, ncols).  Returns binding groups and host copies."""
    groups, host = [], []
    for m, k, nc in specs:
        W, bias = randn(rng, (m, k), np.float32, 0.1), randn(rng, m, np.float32)
        xs = [randn(rng, k, np.float32) for _ in range(nc)]
        dys = [randn(rng, m, np.float32) for _ in range(nc)]
        host.append((W, bias, xs, dys))
        groups.append(dict(w=B.from_host(W), bias=B.from_host(bias),
                           x=[B.from_host(x) for x in xs], dy=[B.from_host(d) for d in dys]))
    return groups, host


@pytest.mark.parametrize("specs", [
    [(8, 5, 1)], [(1024, 384, 7)], [(1024, 384, 256)], [(96, 40, 100), (200, 64, 3), (33, 17, 45)],
    [(1024, 384, 150), (256, 256, 31)],
])
@pytest.mark.parametrize("path", [0, 5])
def test_level_equals_per_node_products(gpu, specs, path):
    """path 0: automatic (equally spaced columns collapse to a strided matrix and may run on
    the TMA-fed kernel); path 5: always through the column tables."""
    gpu.set_option("force_path", path)
    rng = np.random.default_rng(41)
    groups, host = make_level(rng, specs)
    ys = [[torch.zeros(g["w"].shape[0], device="cuda") for _ in g["x"]] for g in groups]
    gpu.grouped(GROUPED_FORWARD, [gpu.Group(w=g["w"], x_cols=g["x"], y_cols=y, bias=g["bias"])
                                  for g, y in zip(groups, ys)])
    dxs = [[torch.ones(g["w"].shape[1], device="cuda") for _ in g["x"]] for g in groups]
    dws = [B.colmajor(*g["w"].shape, torch.float32, fill=1.0) for g in groups]
    dbs = [torch.ones(g["w"].shape[0], device="cuda") for g in groups]
    gpu.grouped(GROUPED_DX, [gpu.Group(w=g["w"], y_cols=g["dy"], dx_cols=dx)
                             for g, dx in zip(groups, dxs)])
    gpu.grouped(GROUPED_DW, [gpu.Group(w=g["w"], x_cols=g["x"], y_cols=g["dy"], dw=dw, dbias=db)
                             for g, dw, db in zip(groups, dws, dbs)])
    torch.cuda.synchronize()
    for (W, bias, xs, dys), y, dx, dw, db in zip(host, ys, dxs, dws, dbs):
        X, DY = np.stack(xs, 1), np.stack(dys, 1)
        check(np.stack([B.to_host(t) for t in y], 1), orc.affine_forward([(W, X)], bias, 0), np.float32, "fwd")
        check(np.stack([B.to_host(t) for t in dx], 1), 1 + orc.gemm(W, DY, trans_a=True), np.float32, "dX")
        check(B.to_host(dw), 1 + orc.gemm(DY, X, trans_b=True), np.float32, "dW")
        check(B.to_host(db), 1 + DY.astype(np.float64).sum(1), np.float32, "dbias")


@pytest.mark.parametrize("dt", [np.float32, np.float16])
def test_reference_elementwise_rule_on_a_level(gpu, dt):
    """Every element of every result of a level within the reference's per-element rule
    (test/check_node.h:104-119), on positive, well-scaled operands as in its own tests."""
    rng = np.random.default_rng(43)
    tdt = torch.float32 if dt == np.float32 else torch.float16
    pos = lambda shape, s: (np.abs(rng.standard_normal(shape)) * s + 0.1 * s).astype(dt)
    specs = [(200, 96, 37), (64, 40, 130)]
    groups, host = [], []
    for m, k, nc in specs:
        W, bias = pos((m, k), 0.02), pos(m, 0.1)
        xs, dys = [pos(k, 1) for _ in range(nc)], [pos(m, 1) for _ in range(nc)]
        host.append((W, bias, xs, dys))
        groups.append(dict(w=B.from_host(W), bias=B.from_host(bias),
                           x=[B.from_host(x) for x in xs], dy=[B.from_host(d) for d in dys]))
    ys = [[torch.zeros(g["w"].shape[0], device="cuda", dtype=tdt) for _ in g["x"]] for g in groups]
    dxs = [[torch.zeros(g["w"].shape[1], device="cuda", dtype=tdt) for _ in g["x"]] for g in groups]
    dws = [B.colmajor(*g["w"].shape, tdt, fill=0.0) for g in groups]
    dbs = [torch.zeros(g["w"].shape[0], device="cuda", dtype=tdt) for g in groups]
    gpu.grouped(GROUPED_FORWARD, [gpu.Group(w=g["w"], x_cols=g["x"], y_cols=y, bias=g["bias"])
                                  for g, y in zip(groups, ys)])
    gpu.grouped(GROUPED_DX, [gpu.Group(w=g["w"], y_cols=g["dy"], dx_cols=dx)
                             for g, dx in zip(groups, dxs)])
    gpu.grouped(GROUPED_DW, [gpu.Group(w=g["w"], x_cols=g["x"], y_cols=g["dy"], dw=dw, dbias=db)
                             for g, dw, db in zip(groups, dws, dbs)])
    torch.cuda.synchronize()
    for (W, bias, xs, dys), y, dx, dw, db in zip(host, ys, dxs, dws, dbs):
        X, DY = np.stack(xs, 1), np.stack(dys, 1)
        check_elementwise(np.stack([B.to_host(t) for t in y], 1), orc.affine_forward([(W, X)], bias, 0), dt, "fwd")
        check_elementwise(np.stack([B.to_host(t) for t in dx], 1), orc.gemm(W, DY, trans_a=True), dt, "dX")
        check_elementwise(B.to_host(dw), orc.gemm(DY, X, trans_b=True), dt, "dW")
        check_elementwise(B.to_host(db), DY.astype(np.float64).sum(1).astype(dt), dt, "dbias")


@pytest.mark.parametrize("dt", [np.float32, np.float16])
@pytest.mark.parametrize("act", [orc.ACT_TANH, orc.ACT_SIGMOID, orc.ACT_RELU])
@pytest.mark.parametrize("layout", ["separate", "matrix"])
def test_level_of_affines_with_a_nonlinearity(gpu, dt, act, layout):
    """What the reference's Autobatch leaves unbatched (ginn/autobatch.h:30-38): Affines with a
    fused nonlinearity.  Forward applies it after the merged product; the gradient launches take
    dy (.) act'(value) as their operand.  Against the per-node Affine of the oracle; columns as
    separate vectors (pointer tables) and as the columns of one matrix (plain products)."""
    rng = np.random.default_rng(61 + act)
    tdt = torch.float32 if dt == np.float32 else torch.float16
    specs = [(200, 96, 37), (64, 40, 130)]
    host, devs = [], []
    for m, k, nc in specs:
        W, bias = randn(rng, (m, k), dt, 0.1), randn(rng, m, dt)
        X, DY = randn(rng, (k, nc), dt), randn(rng, (m, nc), dt)
        host.append((W, bias, X, DY))
        if layout == "matrix":
            Xd, DYd = B.from_host(X), B.from_host(DY)
            Yd, dXd = B.colmajor(m, nc, tdt, fill=0.0), B.colmajor(k, nc, tdt, fill=0.0)
            cols = lambda t: [t[:, j] for j in range(t.shape[1])]
            devs.append((B.from_host(W), B.from_host(bias), cols(Xd), cols(DYd), cols(Yd), cols(dXd)))
        else:
            devs.append((B.from_host(W), B.from_host(bias),
                         [B.from_host(np.ascontiguousarray(X[:, j])) for j in range(nc)],
                         [B.from_host(np.ascontiguousarray(DY[:, j])) for j in range(nc)],
                         [torch.zeros(m, device="cuda", dtype=tdt) for _ in range(nc)],
                         [torch.zeros(k, device="cuda", dtype=tdt) for _ in range(nc)]))
    dws = [B.colmajor(m, k, tdt, fill=0.0) for m, k, _ in specs]
    dbs = [torch.zeros(m, device="cuda", dtype=tdt) for m, _, _ in specs]
    gpu.grouped(GROUPED_FORWARD, [gpu.Group(w=W, x_cols=x, y_cols=y, bias=b, act=act)
                                  for W, b, x, _, y, _ in devs])
    gpu.grouped(GROUPED_DX, [gpu.Group(w=W, y_cols=dy, dx_cols=dx, act=act, out_cols=y)
                             for W, _, _, dy, y, dx in devs])
    gpu.grouped(GROUPED_DW, [gpu.Group(w=W, x_cols=x, y_cols=dy, dw=dw, dbias=db, act=act, out_cols=y)
                             for (W, _, x, dy, y, _), dw, db in zip(devs, dws, dbs)])
    torch.cuda.synchronize()
    for (W, bias, X, DY), (_, _, _, _, y, dx), dw, db in zip(host, devs, dws, dbs):
        Y = np.stack([B.to_host(t) for t in y], 1)
        check(Y, orc.affine_forward([(W, X)], bias, act), dt, "value")
        g = orc.affine_backward([(W, X)], DY, Y, act, dt)
        check(np.stack([B.to_host(t) for t in dx], 1), g["db"][0], dt, "dX")
        check(B.to_host(dw), g["da"][0], dt, "dW")
        check(B.to_host(db), g["dbias"], dt, "dbias")


@pytest.mark.parametrize("prepared", [False, True])
def test_columns_of_one_matrix_need_no_tables(gpu, prepared):
    """The nodes' vectors are the columns of one padded matrix (a batched input, or tensors
    handed out back to back by a bump allocator): the level is then run as plain products.
    Same results as through the tables; both the immediate and the prepared form."""
    rng = np.random.default_rng(47)
    m, k, n, ldx, ldy = 1024, 384, 300, 388, 1024
    W, bias = randn(rng, (m, k), np.float32, 0.05), randn(rng, m, np.float32)
    X, DY = randn(rng, (k, n), np.float32), randn(rng, (m, n), np.float32)
    Wd, bd = B.from_host(W), B.from_host(bias)
    Xd, DYd = B.from_host(X, ld=ldx), B.from_host(DY, ld=ldy)
    cols = lambda t: [t[:, j] for j in range(t.shape[1])]
    results = []
    for path in (0, 5):
        gpu.set_option("force_path", path)
        Y = B.colmajor(m, n, torch.float32, ld=ldy, fill=0.0)
        dX = B.colmajor(k, n, torch.float32, ld=ldx, fill=1.0)
        dW, db = B.colmajor(m, k, torch.float32, fill=1.0), torch.ones(m, device="cuda")
        calls = [(GROUPED_FORWARD, gpu.Group(w=Wd, x_cols=cols(Xd), y_cols=cols(Y), bias=bd)),
                 (GROUPED_DX, gpu.Group(w=Wd, y_cols=cols(DYd), dx_cols=cols(dX))),
                 (GROUPED_DW, gpu.Group(w=Wd, x_cols=cols(Xd), y_cols=cols(DYd), dw=dW, dbias=db))]
        launches = gpu.launch_count()
        for mode, grp in calls:
            if prepared:
                gpu.GroupedCall(mode, [grp])()
            else:
                gpu.grouped(mode, [grp])
        torch.cuda.synchronize()
        assert gpu.launch_count() == launches + 3
        results.append([B.to_host(t) for t in (Y, dX, dW, db)])
    for got in results:
        check(got[0], orc.affine_forward([(W, X)], bias, 0), np.float32, "fwd")
        check(got[1], 1 + orc.gemm(W, DY, trans_a=True), np.float32, "dX")
        check(got[2], 1 + orc.gemm(DY, X, trans_b=True), np.float32, "dW")
        check(got[3], 1 + DY.astype(np.float64).sum(1), np.float32, "dbias")


def test_unaligned_column_vectors(gpu):
    """Columns that are views at odd offsets (what RowwiseUncat produces) take the scalar path."""
    rng = np.random.default_rng(42)
    m, k, nc = 64, 30, 9
    W = randn(rng, (m, k), np.float32)
    pool = torch.zeros(nc * (k + 1) + 1, device="cuda")
    xs_h = [randn(rng, k, np.float32) for _ in range(nc)]
    xs = []
    for j, x in enumerate(xs_h):
        v = pool[1 + j * (k + 1): 1 + j * (k + 1) + k]
        v.copy_(torch.from_numpy(x))
        xs.append(v)
    ys = [torch.zeros(m, device="cuda") for _ in range(nc)]
    gpu.grouped(GROUPED_FORWARD, [gpu.Group(w=B.from_host(W), x_cols=xs, y_cols=ys)])
    torch.cuda.synchronize()
    check(np.stack([B.to_host(t) for t in ys], 1), orc.gemm(W, np.stack(xs_h, 1)), np.float32)


def test_many_levels_reuse_the_staging_ring(gpu):
    rng = np.random.default_rng(43)
    groups, host = make_level(rng, [(128, 64, 20)])
    g = groups[0]
    W, bias, xs, _ = host[0]
    ref = orc.affine_forward([(W, np.stack(xs, 1))], bias, 0)
    for _ in range(300):
        ys = [torch.zeros(128, device="cuda") for _ in xs]
        gpu.grouped(GROUPED_FORWARD, [gpu.Group(w=g["w"], x_cols=g["x"], y_cols=ys, bias=g["bias"])])
    torch.cuda.synchronize()
    check(np.stack([B.to_host(t) for t in ys], 1), ref, np.float32)


def test_prepared_level_equals_one_shot_call_and_survives_reuse(gpu):
    """ginn_b200_level_create / run: same result as ginn_b200_grouped, launch after launch."""
    rng = np.random.default_rng(44)
    groups, host = make_level(rng, [(1024, 384, 33), (96, 40, 7)])
    ys = [[torch.zeros(g["w"].shape[0], device="cuda") for _ in g["x"]] for g in groups]
    level = gpu.GroupedCall(GROUPED_FORWARD, [gpu.Group(w=g["w"], x_cols=g["x"], y_cols=y, bias=g["bias"])
                                              for g, y in zip(groups, ys)])
    for rep in range(3):
        for y in ys:
            for t in y:
                t.fill_(float("nan"))
        level()
        torch.cuda.synchronize()
        for (W, bias, xs, _), y in zip(host, ys):
            check(np.stack([B.to_host(t) for t in y], 1),
                  orc.affine_forward([(W, np.stack(xs, 1))], bias, 0), np.float32, f"rep {rep}")
    dws = [B.colmajor(*g["w"].shape, torch.float32, fill=0.0) for g in groups]
    dbs = [torch.zeros(g["w"].shape[0], device="cuda") for g in groups]
    dw_level = gpu.GroupedCall(GROUPED_DW, [gpu.Group(w=g["w"], x_cols=g["x"], y_cols=g["dy"], dw=dw, dbias=db)
                                            for g, dw, db in zip(groups, dws, dbs)])
    dw_level()
    dw_level()      # gradients accumulate across launches
    torch.cuda.synchronize()
    for (W, bias, xs, dys), dw, db in zip(host, dws, dbs):
        X, DY = np.stack(xs, 1), np.stack(dys, 1)
        check(B.to_host(dw), 2 * orc.gemm(DY, X, trans_b=True), np.float32, "dW")
        check(B.to_host(db), 2 * DY.astype(np.float64).sum(1), np.float32, "dbias")


def test_half_level(gpu):
    """Grouped launches in Half (fp16 gather kernel): forward, dX, dW against the oracle."""
    rng = np.random.default_rng(45)
    m, k, nc = 200, 72, 37
    W, bias = randn(rng, (m, k), np.float16, 0.1), randn(rng, m, np.float16)
    xs, dys = [randn(rng, k, np.float16) for _ in range(nc)], [randn(rng, m, np.float16) for _ in range(nc)]
    Wd, bd = B.from_host(W), B.from_host(bias)
    xd, dyd = [B.from_host(x) for x in xs], [B.from_host(d) for d in dys]
    ys = [torch.zeros(m, device="cuda", dtype=torch.float16) for _ in range(nc)]
    dxs = [torch.zeros(k, device="cuda", dtype=torch.float16) for _ in range(nc)]
    dw = B.colmajor(m, k, torch.float16, fill=0.0)
    db = torch.zeros(m, device="cuda", dtype=torch.float16)
    gpu.grouped(GROUPED_FORWARD, [gpu.Group(w=Wd, x_cols=xd, y_cols=ys, bias=bd)])
    gpu.grouped(GROUPED_DX, [gpu.Group(w=Wd, y_cols=dyd, dx_cols=dxs)])
    gpu.grouped(GROUPED_DW, [gpu.Group(w=Wd, x_cols=xd, y_cols=dyd, dw=dw, dbias=db)])
    torch.cuda.synchronize()
    X, DY = np.stack(xs, 1), np.stack(dys, 1)
    check(np.stack([B.to_host(t) for t in ys], 1), orc.affine_forward([(W, X)], bias, 0), np.float16, "fwd")
    check(np.stack([B.to_host(t) for t in dxs], 1), orc.gemm(W, DY, trans_a=True), np.float16, "dX")
    check(B.to_host(dw), orc.gemm(DY, X, trans_b=True), np.float16, "dW")
    check(B.to_host(db), DY.astype(np.float64).sum(1), np.float16, "dbias")


def test_accumulating_forward_level_with_bias(gpu):
    """y += W x + b into non-zero outputs: the form whose contraction the library may split over
    several CTAs (each adds its partial sum, the first one of a tile also the bias)."""
    rng = np.random.default_rng(46)
    for specs in ([(1024, 384, 256)], [(256, 2048, 40), (128, 96, 7)]):
        groups, host = make_level(rng, specs)
        y0 = [[randn(rng, g["w"].shape[0], np.float32) for _ in g["x"]] for g in groups]
        ys = [[B.from_host(v) for v in col] for col in y0]
        gpu.grouped(GROUPED_FORWARD, [gpu.Group(w=g["w"], x_cols=g["x"], y_cols=y, bias=g["bias"],
                                                accumulate=True) for g, y in zip(groups, ys)])
        torch.cuda.synchronize()
        for (W, bias, xs, _), y, base in zip(host, ys, y0):
            X = np.stack(xs, 1)
            ref = np.stack(base, 1).astype(np.float64) + orc.affine_forward([(W, X)], bias, 0)
            check(np.stack([B.to_host(t) for t in y], 1), ref, np.float32, "y += W x + b")
