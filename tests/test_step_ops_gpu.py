"""GPU parity of the step neighbours (picked negative log softmax, Adam) against the oracle,
through the C ABI."""
import numpy as np
import pytest
import torch

from ginn_b200 import binding as B
from oracle import oracle as orc
from helpers import check, randn

pytestmark = pytest.mark.gpu


def test_pick_nll_known_answer(gpu, kat):
    """test/nodes.cu.cpp:755-797."""
    k = kat["pick_nll"]
    for dt in (np.float32, np.float16):
        x = B.from_host(np.asarray(k["W"], dt))
        idx = torch.tensor(k["index"], dtype=torch.int32, device="cuda")
        smax = B.colmajor(4, 3, x.dtype, fill=0.0)
        val = torch.zeros(3, dtype=x.dtype, device="cuda")
        gpu.pick_nll_forward(x, idx, smax, val)
        torch.cuda.synchronize()
        eps = k["eps"]["f32" if dt == np.float32 else "f16"]
        np.testing.assert_allclose(val.float().cpu().numpy(), k["pnlsm"], rtol=max(eps, 2e-6) * 2)
        np.testing.assert_allclose(B.to_host(smax).astype(np.float64)[k["index"], np.arange(3)],
                                   k["psm"], rtol=max(eps, 2e-6) * 2)


@pytest.mark.parametrize("dt", [np.float32, np.float16])
@pytest.mark.parametrize("rows,cols,pad", [(10, 4096, 0), (1, 7, 0), (33, 100, 3), (1000, 37, 5), (5000, 9, 0)])
def test_pick_nll_forward_backward(gpu, dt, rows, cols, pad):
    """C5's 10 x 4096 logits, a single row, padded leading dimensions, and a vocabulary-sized
    column (one CTA per column)."""
    rng = np.random.default_rng(rows * 131 + cols)
    # Half keeps the picked probability in fp16 before taking its log, as the reference does:
    # logits are kept small enough that no probability falls into the subnormal range
    x = (randn(rng, (rows, cols), dt) * (3 if dt == np.float32 else 0.5)).astype(dt)
    idx = rng.integers(0, rows, cols).astype(np.int32)
    g = randn(rng, (cols,), dt)
    dx0 = randn(rng, (rows, cols), dt)
    X, DX = B.from_host(x, ld=rows + pad), B.from_host(dx0, ld=rows + pad)
    S = B.colmajor(rows, cols, X.dtype, ld=rows + pad, fill=0.0)
    I = torch.from_numpy(idx).cuda()
    V = torch.zeros(cols, dtype=X.dtype, device="cuda")
    G = torch.from_numpy(g).cuda()
    gpu.pick_nll_forward(X, I, S, V)
    gpu.pick_nll_backward(S, I, G, DX)
    torch.cuda.synchronize()
    smax, val = orc.pick_nll_forward(x, idx)
    check(B.to_host(S), smax, dt, "smax")
    check(V.cpu().numpy(), val, dt, "value")
    # backward from the stored (rounded) probabilities, as the node does
    ref = orc.pick_nll_backward(B.to_host(S), idx, g, dx0)
    check(B.to_host(DX), ref, dt, "dx")


@pytest.mark.parametrize("dt", [np.float32, np.float16])
def test_adam_three_steps(gpu, dt):
    """C5's flat parameter buffer size; three steps so that m, v and the bias corrections matter."""
    n = 1_863_690 if dt == np.float32 else 100_003
    rng = np.random.default_rng(77)
    w = randn(rng, (n,), dt)
    m, v = np.zeros(n), np.zeros(n)
    W = torch.from_numpy(w).cuda()
    M = torch.zeros(n, device="cuda")
    Vv = torch.zeros(n, device="cuda")
    wref = w.astype(np.float64)
    for t in (1, 2, 3):
        d = (randn(rng, (n,), dt) * 4).astype(dt)  # some elements beyond the clip of 5
        D = torch.from_numpy(d).cuda()
        gpu.adam_update(W, D, M, Vv, t)
        torch.cuda.synchronize()
        wref, dref, m, v = orc.adam_update(wref, d, m, v, 1e-3, 5.0, 1e-8, 0.9, 0.999, 0.9 ** t, 0.999 ** t)
        wref = wref.astype(dt).astype(np.float64)  # the weight is stored in dt after every step
        np.testing.assert_array_equal(D.cpu().numpy(), dref.astype(dt))
        check(M.cpu().numpy(), m, np.float32, f"m step {t}")
        check(Vv.cpu().numpy(), v, np.float32, f"v step {t}")
        check(W.cpu().numpy(), wref, dt, f"w step {t}")
    if dt == np.float32:
        np.testing.assert_allclose(W.cpu().numpy(), wref, rtol=1e-6, atol=2e-6)  # a few ulp of the largest weights


def test_step_ops_reject_bad_arguments(gpu):
    x = B.colmajor(4, 3, torch.float32, fill=0.0)
    idx = torch.zeros(3, dtype=torch.int32, device="cuda")
    with pytest.raises(B.GinnB200Error):
        B._check(B.lib().ginn_b200_pick_nll_forward(0, None, 0, 4, 3, x.data_ptr(), 2, idx.data_ptr(),
                                                    x.data_ptr(), 4, x.data_ptr()))
    with pytest.raises(B.GinnB200Error):
        B._check(B.lib().ginn_b200_adam_update(0, None, 0, 4, x.data_ptr(), x.data_ptr(), x.data_ptr(),
                                               x.data_ptr(), 1e-3, 5.0, 1e-8, 0.9, 0.999, 1.0, 0.999))


@pytest.mark.parametrize("dt", [np.float32, np.float16])
@pytest.mark.parametrize("shape,pad", [((256, 256, 8), 0), ((3, 5), 0), ((33, 100), 3), ((5000, 6), 0), ((1, 9), 0)])
def test_softmax_forward_backward(gpu, dt, shape, pad):
    """SoftmaxOp (ginn/nonlin.h:157-190) over dimension 0, batches folded into the columns (the
    attention scores of config 3), `=` and `+=` into the input gradient; the reference's own
    softmax values of test/nodes.cu.cpp:755-763 are part of the pick test above."""
    rng = np.random.default_rng(sum(shape))
    x = (randn(rng, shape, dt) * (3 if dt == np.float32 else 1)).astype(dt)
    dy, dx0 = randn(rng, shape, dt), randn(rng, shape, dt)
    ld = shape[0] + pad if len(shape) == 2 else None
    X, DY = B.from_host(x, ld=ld), B.from_host(dy, ld=ld)
    Y = B.from_host(np.zeros(shape, dt), ld=ld)
    gpu.softmax_forward(X, Y)
    torch.cuda.synchronize()
    x2 = x.reshape(shape[0], -1, order="F")
    ref_y = orc.pick_nll_forward(x2, np.zeros(x2.shape[1], np.int64))[0].reshape(shape, order="F")
    check(B.to_host(Y), ref_y, dt, "softmax")
    y_stored = B.to_host(Y).reshape(shape[0], -1, order="F")
    dy2, dx2 = dy.reshape(shape[0], -1, order="F"), dx0.reshape(shape[0], -1, order="F")
    for acc in (False, True):
        DX = B.from_host(dx0, ld=ld)
        gpu.softmax_backward(Y, DY, DX, accumulate=acc)
        torch.cuda.synchronize()
        ref = orc.softmax_backward(y_stored, dy2, dx2 if acc else None)
        check(B.to_host(DX).reshape(shape[0], -1, order="F"), ref, dt, f"dx acc={acc}")


def test_softmax_known_answers(gpu, kat):
    """test/nodes.cu.cpp:689-700 (values) and :728-747 (saturating inputs, -inf, a single row)."""
    k = kat["softmax"]
    for dt, eps in ((np.float32, 1e-5), (np.float16, 2e-3)):
        cases = [(k["W"], k["smaxW"])] + [(c["x"], c["y"]) for c in k["extreme"]]
        for x, y in cases:
            x = np.asarray([[float(v) for v in row] for row in x], dt)
            X = B.from_host(x)
            Y = B.from_host(np.zeros_like(x))
            gpu.softmax_forward(X, Y)
            torch.cuda.synchronize()
            np.testing.assert_allclose(B.to_host(Y).astype(np.float64), np.asarray(y, np.float64),
                                       rtol=eps, atol=eps * 1e-2)


def test_lstm_cell_forward_backward(gpu):
    """The cell update between two autobatch levels: a level with 7 columns of which 4 live on,
    padded leading dimensions, against the fp64 restatement."""
    rng = np.random.default_rng(91)
    H, n, n_next, E = 24, 7, 4, 5
    f32 = np.float32
    G, cp = randn(rng, (4 * H, n), f32), randn(rng, (H, n + 2), f32)
    Gd, CP = B.from_host(G, ld=4 * H + 3), B.from_host(cp)
    C, Hh = B.colmajor(H, n, torch.float32, fill=0.0), B.colmajor(H, n, torch.float32, ld=H + 1, fill=0.0)
    XH = B.colmajor(E + H, n_next, torch.float32, fill=7.0)
    gpu.lstm_cell_forward(Gd, CP, C, Hh, XH[E:], n_next)
    torch.cuda.synchronize()
    act, c, h = orc.lstm_cell_forward(G, cp)
    check(B.to_host(Gd), act, f32, "activations")
    check(B.to_host(C), c, f32, "c")
    check(B.to_host(Hh), h, f32, "h")
    np.testing.assert_array_equal(B.to_host(XH)[:E], 7.0)       # the x block is not touched
    check(B.to_host(XH)[E:], h[:, :n_next], f32, "h copied into the next level's input")
    dhn, dcn = randn(rng, (E + H, n_next), f32), randn(rng, (H, n_next), f32)
    DHN, DCN = B.from_host(dhn), B.from_host(dcn)
    dG, dC = B.colmajor(4 * H, n, torch.float32, fill=0.0), B.colmajor(H, n, torch.float32, fill=0.0)
    gpu.lstm_cell_backward(Gd, C, CP, DHN[E:], DCN, n_next, dG, dC, dh_end=1.0)
    torch.cuda.synchronize()
    rg, rc = orc.lstm_cell_backward(B.to_host(Gd), B.to_host(C), cp, dhn[E:], dcn, n_next, 1.0)
    check(B.to_host(dG), rg, f32, "dgates")
    check(B.to_host(dC), rc, f32, "dc")
    # first level (no previous cell state) and last level (no column lives on)
    C0 = B.colmajor(H, n, torch.float32, fill=0.0)
    G0 = B.from_host(G)
    gpu.lstm_cell_forward(G0, None, C0, Hh, None, 0)
    gpu.lstm_cell_backward(G0, C0, None, None, None, 0, dG, dC, dh_end=0.5)
    torch.cuda.synchronize()
    act0, c0, _ = orc.lstm_cell_forward(G, None)
    rg0, rc0 = orc.lstm_cell_backward(act0, c0, None, None, None, 0, 0.5)
    check(B.to_host(dG), rg0, f32, "dgates, no neighbours")
    check(B.to_host(dC), rc0, f32, "dc, no neighbours")


def test_lstm_cells_over_per_cell_tensors(gpu):
    """The cell update with every cell in tensors of its own (one graph node per sequence and
    step): same arithmetic as the matrix form, gradients accumulated (+=), a cell without a
    predecessor in the same launch.  Against the fp64 restatement."""
    rng = np.random.default_rng(92)
    H, n = 24, 6
    f32 = np.float32
    G, cp = randn(rng, (4 * H, n), f32), randn(rng, (H, n), f32)
    cp[:, 2] = 0.0                                     # cell 2 starts a sequence: no c_prev
    dev = lambda a: [B.from_host(np.ascontiguousarray(a[:, j])) for j in range(a.shape[1])]
    zeros = lambda r: [torch.zeros(r, device="cuda") for _ in range(n)]
    Gs, CPs, Cs, Hs = dev(G), dev(cp), zeros(H), zeros(H)
    CPs[2] = None
    gpu.lstm_cells(False, [Gs, CPs, Cs, Hs])
    torch.cuda.synchronize()
    stack = lambda ts: np.stack([B.to_host(t) for t in ts], 1)
    act, c, h = orc.lstm_cell_forward(G, cp)
    check(stack(Gs), act, f32, "activations")
    check(stack(Cs), c, f32, "c")
    check(stack(Hs), h, f32, "h")
    dh, dc = randn(rng, (H, n), f32), randn(rng, (H, n), f32)
    dGs = [torch.full((4 * H,), 0.5, device="cuda") for _ in range(n)]
    dCPs = [torch.full((H,), 0.25, device="cuda") for _ in range(n)]
    dCPs[2] = None
    gpu.lstm_cells(True, [Gs, Cs, CPs, dev(dh), dev(dc), dGs, dCPs])
    torch.cuda.synchronize()
    rg, rc = orc.lstm_cell_backward(stack(Gs), stack(Cs), cp, dh, dc, n, 0.0)
    check(stack(dGs), 0.5 + rg, f32, "dgates +=")
    keep = [j for j in range(n) if j != 2]
    check(stack([dCPs[j] for j in keep]), 0.25 + rc[:, keep], f32, "dc_prev +=")


@pytest.mark.parametrize("tdt", [torch.float32, torch.float16])
def test_fill(gpu, tdt):
    x = torch.zeros(100003, device="cuda", dtype=tdt)
    gpu.fill(x, 0.375)
    torch.cuda.synchronize()
    assert bool((x == 0.375).all())
