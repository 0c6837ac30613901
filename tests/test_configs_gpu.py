"""Parity at the full sizes of the benchmark configurations (all through the C ABI):
   config 2  autobatched LSTM gates, 256 sequences of length 5..40, W 1024 x 384
   config 3  min-GPT attention through BatchedProd, 256 batches of 256 x 64 x 256
   config 5  the three Affine layers of the MLP at batch 4096
Inputs are seeded synthetic data of the configurations' shapes and distributions; the oracle
is the fp64 restatement in oracle/oracle.py."""
import numpy as np
import pytest
import torch

from oracle import oracle as orc
from ginn_b200 import binding as B
from ginn_b200.binding import GROUPED_DW, GROUPED_DX, GROUPED_FORWARD
from helpers import check, randn

pytestmark = pytest.mark.gpu


def test_config3_attention_products(gpu):
    rng = np.random.default_rng(20243)
    T, hs, nb = 256, 64, 256
    sd = np.sqrt(1 / 8)
    k = randn(rng, (T, hs, nb), np.float32, sd)     # K' : T x hs per (batch, head)
    q = randn(rng, (hs, T, nb), np.float32, sd)
    v = randn(rng, (hs, T, nb), np.float32, sd)
    d_o = randn(rng, (hs, T, nb), np.float32)
    kd, qd, vd, dod = map(B.from_host, (k, q, v, d_o))
    S = B.colmajor(T, T, torch.float32, batches=nb, fill=0.0)
    gpu.gemm_batched(kd, qd, S)                                      # scores = K' * Q
    torch.cuda.synchronize()
    s_host = B.to_host(S)
    check(s_host, orc.gemm_batched(k, q), np.float32, "scores")
    P = B.colmajor(T, T, torch.float32, batches=nb)
    P.copy_(torch.softmax(S, dim=0))                                 # column softmax (glue)
    O = B.colmajor(hs, T, torch.float32, batches=nb, fill=0.0)
    gpu.gemm_batched(vd, P, O)                                       # out = V * P
    torch.cuda.synchronize()
    p_host = B.to_host(P)
    check(B.to_host(O), orc.gemm_batched(v, p_host), np.float32, "out")
    # backward: dV += dO * P^T, dP += V^T * dO, then (through the softmax) dK' and dQ
    dV = B.colmajor(hs, T, torch.float32, batches=nb, fill=0.0)
    dP = B.colmajor(T, T, torch.float32, batches=nb, fill=0.0)
    gpu.gemm_batched(dod, P, dV, trans_b=True, accumulate=True)
    gpu.gemm_batched(vd, dod, dP, trans_a=True, accumulate=True)
    dS = B.colmajor(T, T, torch.float32, batches=nb)
    dS.copy_(P * (dP - (P * dP).sum(dim=0, keepdim=True)))           # softmax backward (glue)
    dK = B.colmajor(T, hs, torch.float32, batches=nb, fill=0.0)
    dQ = B.colmajor(hs, T, torch.float32, batches=nb, fill=0.0)
    gpu.gemm_batched(dS, qd, dK, trans_b=True, accumulate=True)
    gpu.gemm_batched(kd, dS, dQ, trans_a=True, accumulate=True)
    torch.cuda.synchronize()
    ds_host = B.to_host(dS)
    check(B.to_host(dV), orc.gemm_batched(d_o, p_host, trans_b=True), np.float32, "dV")
    check(B.to_host(dP), orc.gemm_batched(v, d_o, trans_a=True), np.float32, "dP")
    check(B.to_host(dK), orc.gemm_batched(ds_host, q, trans_b=True), np.float32, "dK")
    check(B.to_host(dQ), orc.gemm_batched(k, ds_host, trans_a=True), np.float32, "dQ")


def xavier(rng, rows, cols):
    a = np.sqrt(6 / (0.5 * (rows + cols)))                           # ginn/init/init.h:45-51
    return rng.uniform(-a, a, (rows, cols)).astype(np.float32)


def test_config5_mlp_layers_forward_backward(gpu):
    rng = np.random.default_rng(20245)
    batch = 4096
    dims = [784, 1024, 1024, 10]
    acts = [gpu.ACT_RELU, gpu.ACT_RELU, gpu.ACT_NONE]
    Ws = [xavier(rng, dims[i + 1], dims[i]) for i in range(3)]
    bs = [xavier(rng, dims[i + 1], 1).ravel() for i in range(3)]
    x = rng.uniform(0, 1, (784, batch)).astype(np.float32)
    labels = rng.integers(0, 10, batch)
    Wd, bd = [B.from_host(w) for w in Ws], [B.from_host(b) for b in bs]
    h = [B.from_host(x)]
    for i in range(3):
        y = B.colmajor(dims[i + 1], batch, torch.float32, fill=0.0)
        gpu.affine_forward([gpu.Pair(Wd[i], h[-1])], bd[i], acts[i], y)
        h.append(y)
    torch.cuda.synchronize()
    # oracle forward, layer by layer from the GPU's own inputs (as the CPU-vs-GPU protocol does)
    hh = [x] + [B.to_host(t) for t in h[1:]]
    for i in range(3):
        check(hh[i + 1], orc.affine_forward([(Ws[i], hh[i])], bs[i], acts[i]), np.float32, f"layer {i}")
    # loss = sum over the batch of -log softmax(logits)[label]   (glue), gradient wrt logits
    logits = hh[3].astype(np.float64)
    p = np.exp(logits - logits.max(0))
    p /= p.sum(0)
    dlog = p.copy()
    dlog[labels, np.arange(batch)] -= 1
    dy = B.from_host(dlog.astype(np.float32))
    dyh = dlog.astype(np.float32)
    for i in (2, 1, 0):
        dW = B.colmajor(dims[i + 1], dims[i], torch.float32, fill=0.0)
        db = torch.zeros(dims[i + 1], device="cuda")
        dX = B.colmajor(dims[i], batch, torch.float32, fill=0.0) if i > 0 else None
        gpu.affine_backward([gpu.PairGrad(Wd[i], h[i], dW, dX)], dy, h[i + 1], acts[i], db)
        torch.cuda.synchronize()
        g = orc.affine_backward([(Ws[i], hh[i])], dyh, hh[i + 1], acts[i], np.float32)
        check(B.to_host(dW), g["da"][0], np.float32, f"dW{i}")
        check(B.to_host(db), g["dbias"], np.float32, f"db{i}")
        if i > 0:
            check(B.to_host(dX), g["db"][0], np.float32, f"dX{i}")
            dy, dyh = dX, B.to_host(dX)


def test_config2_lstm_gate_levels(gpu):
    """Recurrent variant: per sequence and step gates = Affine(W, [x_t; h_{t-1}], b); step t of
    every live sequence is one grouped launch.  Each level is checked against the per-node
    Affines of the un-batched graph (the before/after protocol of test/autobatch.cpp)."""
    rng = np.random.default_rng(20242)
    nseq, H, E = 256, 256, 128
    lens = rng.integers(5, 41, nseq)
    W = xavier(rng, 4 * H, E + H)
    b = xavier(rng, 4 * H, 1).ravel()
    Wd, bd = B.from_host(W), B.from_host(b)
    dW = B.colmajor(4 * H, E + H, torch.float32, fill=0.0)
    db = torch.zeros(4 * H, device="cuda")
    dW_ref, db_ref = np.zeros((4 * H, E + H)), np.zeros(4 * H)
    h = {s: torch.randn(H, device="cuda") for s in range(nseq)}
    c = {s: torch.zeros(H, device="cuda") for s in range(nseq)}
    for t in range(int(lens.max())):
        live = [s for s in range(nseq) if lens[s] > t]
        xh = [torch.cat([torch.randn(E, device="cuda"), h[s]]) for s in live]   # [x_t; h_{t-1}]
        gates = [torch.empty(4 * H, device="cuda") for _ in live]
        gpu.grouped(GROUPED_FORWARD, [gpu.Group(w=Wd, x_cols=xh, y_cols=gates, bias=bd)])
        torch.cuda.synchronize()
        XH = np.stack([B.to_host(v) for v in xh], 1)
        G = np.stack([B.to_host(g) for g in gates], 1)
        check(G, orc.affine_forward([(W, XH)], b, orc.ACT_NONE), np.float32, f"level {t}")
        # LSTM cell update (glue), gate order i, f, g, o
        for s, g in zip(live, gates):
            i_, f_, g_, o_ = g[:H], g[H:2 * H], g[2 * H:3 * H], g[3 * H:]
            c[s] = torch.sigmoid(f_) * c[s] + torch.sigmoid(i_) * torch.tanh(g_)
            h[s] = torch.sigmoid(o_) * torch.tanh(c[s])
        if t in (0, 7, int(lens.max()) - 1):     # backward products of a few levels
            dg = [torch.randn(4 * H, device="cuda") for _ in live]
            dxh = [torch.zeros(E + H, device="cuda") for _ in live]
            gpu.grouped(GROUPED_DX, [gpu.Group(w=Wd, y_cols=dg, dx_cols=dxh)])
            gpu.grouped(GROUPED_DW, [gpu.Group(w=Wd, x_cols=xh, y_cols=dg, dw=dW, dbias=db)])
            torch.cuda.synchronize()
            DG = np.stack([B.to_host(v) for v in dg], 1).astype(np.float64)
            check(np.stack([B.to_host(v) for v in dxh], 1), W.astype(np.float64).T @ DG, np.float32, "dX")
            dW_ref += DG @ XH.astype(np.float64).T
            db_ref += DG.sum(1)
    check(B.to_host(dW), dW_ref, np.float32, "dW over levels")
    check(B.to_host(db), db_ref, np.float32, "db over levels")


@pytest.mark.parametrize("fused_cell", [True, False])
def test_lstm_harness_matches_autograd(gpu, fused_cell):
    """The benchmark's autobatched LSTM harness (grouped launches + the cell update, as one
    kernel per level or as torch ops) against torch autograd in fp64 on the same small problem:
    dW and db of the shared gate weights."""
    from ginn_b200.workloads import LstmAutobatch
    w = LstmAutobatch(torch.device("cuda", 0), nseq=9, H=32, E=16, seed=3, fused_cell=fused_cell)
    w.rewrite()
    w.step()
    torch.cuda.synchronize()
    H, E = w.H, w.E
    W = w.W.double().clone().requires_grad_(True)
    b = w.b.double().clone().requires_grad_(True)
    h = w.XH[0][E:].double()
    c = torch.zeros(H, w.n[0], dtype=torch.float64, device="cuda")
    loss = 0.0
    for t in range(w.T):
        n = w.n[t]
        xh = torch.cat([w.XH[t][:E].double(), h[:, :n]], 0)
        G = W @ xh + b[:, None]
        i, f, g, o = torch.sigmoid(G[:H]), torch.sigmoid(G[H:2 * H]), torch.tanh(G[2 * H:3 * H]), torch.sigmoid(G[3 * H:])
        c = f * c[:, :n] + i * g
        h = o * torch.tanh(c)
        ends = w.n[t + 1] if t + 1 < w.T else 0
        loss = loss + h[:, ends:].sum()
    loss.backward()
    check(B.to_host(w.dW), W.grad.cpu().numpy(), np.float32, "dW")
    check(B.to_host(w.db), b.grad.cpu().numpy(), np.float32, "db")


def test_mlp_harness_matches_autograd_and_adam(gpu):
    """Config 5's training step (three fused Affines, picked negative log softmax, Adam in one
    kernel each) against torch autograd in fp64 and a restatement of ginn's Adam
    (ginn/update/update.h:115-133).  Each step starts the fp64 side from the GPU's current
    parameters and feeds its Adam the GPU's (clipped) gradients: Adam's first steps move a weight
    by about lr * sign(gradient), so a gradient that is zero to rounding would otherwise decide
    the comparison."""
    from ginn_b200.workloads import MlpDataParallel
    w = MlpDataParallel(torch.device("cuda", 0), batch=256)
    views = list(w.W) + list(w.b)
    gviews = list(w.dW) + list(w.db)
    m = [torch.zeros_like(p, dtype=torch.float64) for p in views]
    v = [torch.zeros_like(p, dtype=torch.float64) for p in views]
    x = w.x.double()
    for t in (1, 2, 3):
        params = [p.double().clone().requires_grad_(True) for p in views]
        w.step()
        torch.cuda.synchronize()
        h = x
        for i in range(3):
            h = params[i] @ h + params[3 + i][:, None]
            if i < 2:
                h = torch.relu(h)
        loss = torch.nn.functional.cross_entropy(h.T, w.labels, reduction="sum")
        loss.backward()
        assert abs(float(w.loss) - float(loss)) <= 1e-5 * abs(float(loss))
        with torch.no_grad():
            for i, p in enumerate(params):
                g = p.grad.clamp(-5.0, 5.0)
                got = gviews[i].double()
                assert float((got - g).norm() / g.norm()) <= 1e-5, f"gradient {i} step {t}"
                m[i] = 0.9 * m[i] + 0.1 * got
                v[i] = 0.999 * v[i] + 0.001 * got * got
                want = p + (-1e-3 / (1 - 0.9 ** t)) * m[i] / (1e-8 + (v[i] / (1 - 0.999 ** t)).sqrt())
                now = views[i].double()
                assert float((now - want).norm() / want.norm()) <= 1e-6, f"parameter {i} step {t}"


def test_mlp_step_replayed_from_graphs_matches_the_launched_step(gpu):
    """The two CUDA graphs that replay a step's kernel launches must leave the loss, the gradients
    and the parameters where the call-by-call step leaves them (not bit for bit: products whose
    contraction is split over CTAs add their parts in the order the CTAs finish)."""
    from ginn_b200.workloads import MlpDataParallel
    dev = torch.device("cuda", 0)
    a, b = MlpDataParallel(dev, batch=512), MlpDataParallel(dev, batch=512)
    assert torch.equal(a.params, b.params)
    a.step()
    b.step()
    b.capture()
    for _ in range(3):
        a.step()
        b.step()
    torch.cuda.synchronize()
    rel = lambda x, y: float((x.double() - y.double()).norm() / y.double().norm())
    assert abs(float(a.loss) - float(b.loss)) <= 1e-6 * abs(float(a.loss))
    assert rel(b.grads, a.grads) <= 1e-5
    assert rel(b.params, a.params) <= 1e-5
