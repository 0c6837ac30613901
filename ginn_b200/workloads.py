"""Harnesses for the benchmark configurations other than the large Half product.

Each harness builds seeded synthetic inputs of its configuration's shapes, drives the products
through the C ABI (ginn_b200.binding) and keeps everything that is not a matrix product --
softmax, LSTM cell arithmetic, cross-entropy, Adam -- as plain torch elementwise "glue", which is
excluded from the flop counts.  bench.py selects them with --workload.
"""
from __future__ import annotations

import math

import torch

from . import binding as B
from .binding import GROUPED_DW, GROUPED_DX, GROUPED_FORWARD


def _xavier(rows, cols, gen, device):
    """ginn's Xavier: U(-a, a), a = sqrt(6 / (0.5 (rows + cols)))  (ginn/init/init.h:45-51)."""
    a = math.sqrt(6.0 / (0.5 * (rows + cols)))
    buf = (torch.rand(cols, rows, device=device, generator=gen) * 2 - 1) * a
    return buf.T  # column-major rows x cols


def graphed(step):
    """Records one call of `step` into a CUDA graph and returns the replay function.  For steps
    whose launches the host cannot issue as fast as the GPU runs them (a handful of small
    kernels): the replay shows the device time.  `step` must make no allocation and pass the
    same scalars every time."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        step()  # library state (function attributes, contexts) warm before the capture
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        step()
    return g.replay


class AffineLayer:
    """One AffineNode forward + backward with tanh through the fused entry points (config 1 at
    m, n, k = 512, 128, 784; config 5's hidden layer at 1024, 4096, 1024).  Gradients are zeroed
    every step, as Graph::reset_grad does."""

    def __init__(self, device, m, n, k, half=False, seed=20241):
        g = torch.Generator(device=device).manual_seed(seed)
        tdt = torch.float16 if half else torch.float32
        self.W = _xavier(m, k, g, device).to(tdt)
        self.X = torch.randn(n, k, device=device, generator=g).to(tdt).T
        self.b = _xavier(m, 1, g, device).reshape(-1).contiguous().to(tdt)
        self.dY = torch.randn(n, m, device=device, generator=g).to(tdt).T
        self.Y = B.colmajor(m, n, tdt, device, fill=0.0)
        # dW | dX | db in one buffer (16-byte aligned pieces), so that reset_grad is one fill
        pad = lambda c: (c + 7) // 8 * 8
        o_x, o_b = pad(m * k), pad(m * k) + pad(k * n)
        self.grads = torch.zeros(o_b + m, device=device, dtype=tdt)
        self.dW = torch.as_strided(self.grads, (m, k), (1, m))
        self.dX = torch.as_strided(self.grads, (k, n), (1, k), o_x)
        self.db = self.grads[o_b:o_b + m]
        # the node's d-pre-activation tensor (ginn/node/affine.h:82): the Half path writes it
        self.dpre = B.colmajor(m, n, tdt, device, fill=0.0) if half else None
        self.flops = 3 * 2 * m * n * k
        self.units = 1

    def step(self):
        self.grads.zero_()
        B.affine_forward([B.Pair(self.W, self.X)], self.b, B.ACT_TANH, self.Y)
        B.affine_backward([B.PairGrad(self.W, self.X, self.dW, self.dX)], self.dY, self.Y,
                          B.ACT_TANH, self.db, self.dpre)


class Attention:
    """Config 3: min-GPT attention through BatchedProd (examples/min-gpt.cu.cpp:108-157):
    S = K' * Q, column softmax, O = V * P, and the four backward products; 256 (batch, head)
    pairs, T = 256, head size 64, fp32."""

    def __init__(self, device, T=256, hs=64, nb=256, seed=20243, fused=True):
        self.fused = fused
        g = torch.Generator(device=device).manual_seed(seed)
        sd = math.sqrt(1 / 8)

        def cm(r, c, scale=1.0):
            t = B.colmajor(r, c, torch.float32, device, batches=nb)
            t.copy_(torch.randn(r, c, nb, device=device, generator=g) * scale)
            return t

        self.k, self.q, self.v = cm(T, hs, sd), cm(hs, T, sd), cm(hs, T, sd)
        self.dO = cm(hs, T)
        z = lambda r, c: B.colmajor(r, c, torch.float32, device, batches=nb, fill=0.0)
        self.S, self.P, self.dP, self.dS = z(T, T), z(T, T), z(T, T), z(T, T)
        self.O = z(hs, T)
        # the three gradients in one allocation (a PreallocGpu slab hands them out back to back):
        # reset_grad is one fill
        n = hs * T * nb
        self.grads = torch.zeros(3 * n, device=device)
        as3 = lambda off, r, c: torch.as_strided(self.grads, (r, c, nb), (1, r, r * c), off)
        self.dV, self.dQ, self.dK = as3(0, hs, T), as3(n, hs, T), as3(2 * n, T, hs)
        self.flops = 6 * nb * 2 * T * hs * T
        self.units = nb

    def step(self):
        gb = B
        if self.fused:
            # one kernel forward (scores stay on the SM; P is kept for the backward pass), then
            # the composed backward: four batched products and one softmax-backward pass
            self.grads.zero_()
            gb.attention_forward(self.k, self.q, self.v, self.O, self.P)
            gb.attention_backward(self.k, self.q, self.v, self.P, self.dO, self.dS, self.dK, self.dQ,
                                  self.dV)
            return
        self.grads.zero_()
        self.dP.zero_()
        gb.gemm_batched(self.k, self.q, self.S)
        gb.softmax_forward(self.S, self.P)  # SoftmaxOp::forward, ginn/nonlin.h:162-168
        gb.gemm_batched(self.v, self.P, self.O)
        gb.gemm_batched(self.dO, self.P, self.dV, trans_b=True, accumulate=True)
        gb.gemm_batched(self.v, self.dO, self.dP, trans_a=True, accumulate=True)
        gb.softmax_backward(self.P, self.dP, self.dS, accumulate=False)  # nonlin.h:169-190
        gb.gemm_batched(self.dS, self.q, self.dK, trans_b=True, accumulate=True)
        gb.gemm_batched(self.k, self.dS, self.dQ, trans_a=True, accumulate=True)


class LstmAutobatch:
    """Config 2 (recurrent variant): `nseq` sequences of length U{5..40}; per sequence and step
    gates = Affine(W, [x_t; h_{t-1}], b) with one shared W (4H x (E+H)) -- the graph ginn's
    Autobatch turns into one merged product per step.  Step t of every live sequence is one
    grouped launch (forward, dX, dW); every column is addressed through the pointer tables, as the
    nodes' own tensors would be.  Loss = sum of the final hidden states."""

    def __init__(self, device, nseq=256, H=256, E=128, seed=20242, static=False, fused_cell=True):
        g = torch.Generator(device=device).manual_seed(seed)
        cpu_g = torch.Generator().manual_seed(seed)
        lens = torch.randint(5, 41, (nseq,), generator=cpu_g).sort(descending=True).values
        self.lens, self.H, self.E, self.nseq = lens, H, E, nseq
        self.T = int(lens.max())
        self.n = [int((lens > t).sum()) for t in range(self.T)]  # live sequences = a prefix
        self.nodes = int(lens.sum())
        self.W = _xavier(4 * H, E + H, g, device)
        self.b = _xavier(4 * H, 1, g, device).reshape(-1).contiguous()
        # Gradients are carved from flat buffers, as the nodes' tensors are from a PreallocGpu
        # slab (ginn/dev.h:216-251): reset_grad is then a few large fills instead of one per
        # tensor (forty-three 2.4 us kernels on the critical path of a 0.75 ms step).
        self.dWb = torch.zeros(4 * H * (E + H) + 4 * H, device=device)
        self.dW = torch.as_strided(self.dWb, (4 * H, E + H), (1, 4 * H))
        self.db = self.dWb[4 * H * (E + H):]
        cm = lambda r, c: B.colmajor(r, c, torch.float32, device, fill=0.0)
        self.XH = [cm(E + H, n) for n in self.n]
        self.dXflat = torch.zeros((E + H) * sum(self.n), device=device)
        self.dXH, off = [], 0
        for n in self.n:
            self.dXH.append(torch.as_strided(self.dXflat, (E + H, n), (1, E + H), off))
            off += (E + H) * n
        # The gate matrices of all levels share one buffer that is zeroed once per step: the
        # forward products then accumulate (y += W x + b), which lets the library split their
        # contraction over several CTAs (a level has only 16 output tiles and 12 k-blocks).
        self.Gflat = torch.zeros(4 * H * sum(self.n), device=device)
        self.G, off = [], 0
        for n in self.n:
            self.G.append(torch.as_strided(self.Gflat, (4 * H, n), (1, 4 * H), off))
            off += 4 * H * n
        self.dG = [cm(4 * H, n) for n in self.n]
        self.c = [cm(H, n) for n in self.n]
        self.h = [cm(H, n) for n in self.n]
        for t in range(self.T):
            self.XH[t][:E].copy_(torch.randn(E, self.n[t], device=device, generator=g))
        self.XH[0][E:].copy_(torch.randn(H, self.n[0], device=device, generator=g))
        self.flops = 3 * 2 * 4 * H * (E + H) * self.nodes
        self.units = self.nodes
        self.static = static
        # The elementwise cell update between the levels: one kernel per level and pass, or the
        # same arithmetic as a sequence of torch ops (kept as a cross-check of the kernel).
        self.fused_cell = fused_cell
        self.dc = [cm(H, n) for n in self.n]
        self.side = None
        self.fwd = self.dx = self.dw = None
        self.graph = None

    def rewrite(self):
        """The host-side part of autobatching: one prepared grouped call per level and pass."""
        cols = lambda m: [m[:, j] for j in range(m.shape[1])]
        mk = lambda mode, grp: B.GroupedCall(mode, [grp], static=self.static)
        self.fwd, self.dx, self.dw = [], [], []
        for t in range(self.T):
            x, y, dy, dx = cols(self.XH[t]), cols(self.G[t]), cols(self.dG[t]), cols(self.dXH[t])
            self.fwd.append(mk(GROUPED_FORWARD, B.Group(w=self.W, x_cols=x, y_cols=y, bias=self.b,
                                                        accumulate=True)))
            self.dx.append(mk(GROUPED_DX, B.Group(w=self.W, y_cols=dy, dx_cols=dx)))
            self.dw.append(mk(GROUPED_DW, B.Group(w=self.W, x_cols=x, y_cols=dy, dw=self.dW,
                                                  dbias=self.db)))
        # Argument lists of the cell-update calls, built once (slot 1 is the stream): a step
        # launched from Python is bound by host time per call.
        H, E, dev = self.H, self.E, B._dev(self.W)
        ptr = lambda t: None if t is None else t.data_ptr()
        ld = lambda t: 0 if t is None else B._ld(t)
        self.cf_args, self.cb_args = [], []
        for t in range(self.T):
            nxt = self.n[t + 1] if t + 1 < self.T else 0
            cp = self.c[t - 1] if t > 0 else None
            xh = self.XH[t + 1][E:] if nxt else None
            self.cf_args.append([dev, None, H, self.n[t], nxt, ptr(self.G[t]), ld(self.G[t]), ptr(cp), ld(cp),
                                 ptr(self.c[t]), ld(self.c[t]), ptr(self.h[t]), ld(self.h[t]), ptr(xh), ld(xh)])
            dhn = self.dXH[t + 1][E:] if nxt else None
            dcn = self.dc[t + 1] if nxt else None
            self.cb_args.append([dev, None, H, self.n[t], nxt, ptr(self.G[t]), ld(self.G[t]), ptr(self.c[t]),
                                 ld(self.c[t]), ptr(cp), ld(cp), ptr(dhn), ld(dhn), ptr(dcn), ld(dcn), 1.0,
                                 ptr(self.dG[t]), ld(self.dG[t]), ptr(self.dc[t]), ld(self.dc[t])])
        self.events = [torch.cuda.Event() for _ in range(self.T)]

    def forward(self):
        H, E = self.H, self.E
        self.gates = []
        self.Gflat.zero_()
        if self.fused_cell:
            st = torch.cuda.current_stream().cuda_stream
            cell, check = B.lib().ginn_b200_lstm_cell_forward, B._check
            for t in range(self.T):
                self.fwd[t].run(st)
                a = self.cf_args[t]
                a[1] = st
                check(cell(*a))
            return
        for t in range(self.T):
            self.fwd[t]()
            G, n = self.G[t], self.n[t]
            i, f, gg, o = (torch.sigmoid(G[:H]), torch.sigmoid(G[H:2 * H]), torch.tanh(G[2 * H:3 * H]),
                           torch.sigmoid(G[3 * H:]))
            c_prev = self.c[t - 1][:, :n] if t > 0 else torch.zeros_like(self.c[t])
            self.c[t].copy_(f * c_prev + i * gg)
            tc = torch.tanh(self.c[t])
            self.h[t].copy_(o * tc)
            self.gates.append((i, f, gg, o, tc, c_prev))
            if t + 1 < self.T:
                self.XH[t + 1][E:].copy_(self.h[t][:, :self.n[t + 1]])

    def reset_grad(self):
        self.dWb.zero_()
        self.dXflat.zero_()

    def backward(self):
        H, E = self.H, self.E
        if self.fused_cell:
            # The weight-gradient product of a level is needed by nothing before the end of the
            # pass: it runs on a side stream (a parallel branch when captured in a CUDA graph),
            # off the chain cell update -> input gradient -> previous level.  The side stream
            # keeps the accumulations into dW in order.
            main = torch.cuda.current_stream()
            if self.side is None:
                self.side = torch.cuda.Stream(device=self.W.device)
            st, side_st = main.cuda_stream, self.side.cuda_stream
            cell, check = B.lib().ginn_b200_lstm_cell_backward, B._check
            for t in reversed(range(self.T)):
                a = self.cb_args[t]
                a[1] = st
                check(cell(*a))
                ready = self.events[t]
                ready.record(main)
                self.dx[t].run(st)
                self.side.wait_event(ready)
                self.dw[t].run(side_st)
            main.wait_stream(self.side)
            return
        dh_next = dc_next = None  # gradients flowing from step t+1 (a prefix of the columns)
        for t in reversed(range(self.T)):
            n = self.n[t]
            i, f, gg, o, tc, c_prev = self.gates[t]
            dh = torch.zeros(H, n, device=self.W.device)
            dc = torch.zeros(H, n, device=self.W.device)
            if dh_next is not None:
                dh[:, :dh_next.shape[1]] += dh_next
                dc[:, :dc_next.shape[1]] += dc_next
            ends = self.n[t + 1] if t + 1 < self.T else 0
            dh[:, ends:] += 1.0                      # sequences that end here feed the loss
            dc = dc + dh * o * (1 - tc * tc)
            dG = self.dG[t]
            dG[:H].copy_(dc * gg * i * (1 - i))
            dG[H:2 * H].copy_(dc * c_prev * f * (1 - f))
            dG[2 * H:3 * H].copy_(dc * i * (1 - gg * gg))
            dG[3 * H:].copy_(dh * tc * o * (1 - o))
            self.dx[t]()
            self.dw[t]()
            dh_next, dc_next = self.dXH[t][E:], dc * f

    def step(self):
        if self.graph is not None:
            self.graph.replay()
            return
        self.forward()
        self.reset_grad()
        self.backward()

    def capture(self):
        """Records one forward + reset_grad + backward pass (prepared levels and glue) into a CUDA
        graph; later steps replay it.  The prepared levels make no host-to-device copies, so
        the capture holds only kernel launches."""
        assert not self.static, "the allocation-free grouped entry point refuses stream capture"
        self.graph = None
        side = torch.cuda.Stream(device=self.W.device)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            self.step()  # warm up allocator and library state outside the capture
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            self.forward()
            self.reset_grad()
            self.backward()
        self.graph = g


class LstmFlat:
    """Config 2, flat variant: the hidden states are independent data too, so all sum(len) gate
    Affines share one height and autobatch merges them into a single level: one grouped launch per
    pass with sum(len) gathered columns.  Isolates the grouped kernel's throughput from the
    latency of 40 dependent levels."""

    def __init__(self, device, nseq=256, H=256, E=128, seed=20242):
        g = torch.Generator(device=device).manual_seed(seed)
        cpu_g = torch.Generator().manual_seed(seed)
        lens = torch.randint(5, 41, (nseq,), generator=cpu_g)
        self.nodes = n = int(lens.sum())
        self.W = _xavier(4 * H, E + H, g, device)
        self.b = _xavier(4 * H, 1, g, device).reshape(-1).contiguous()
        # all gradients in one buffer (dW | db | dXH), so that reset_grad is one fill
        n_w, n_b = 4 * H * (E + H), 4 * H
        self.grads = torch.zeros(n_w + n_b + (E + H) * n, device=device)
        self.dW = torch.as_strided(self.grads[:n_w], (4 * H, E + H), (1, 4 * H))
        self.db = self.grads[n_w:n_w + n_b]
        self.XH = B.colmajor(E + H, n, torch.float32, device)
        self.XH.copy_(torch.randn(E + H, n, device=device, generator=g))
        self.dG = B.colmajor(4 * H, n, torch.float32, device)
        self.dG.copy_(torch.randn(4 * H, n, device=device, generator=g))
        self.G = B.colmajor(4 * H, n, torch.float32, device, fill=0.0)
        self.dXH = torch.as_strided(self.grads[n_w + n_b:], (E + H, n), (1, E + H))
        cols = lambda m: [m[:, j] for j in range(m.shape[1])]
        x, y, dy, dx = cols(self.XH), cols(self.G), cols(self.dG), cols(self.dXH)
        self.fwd = B.GroupedCall(GROUPED_FORWARD, [B.Group(w=self.W, x_cols=x, y_cols=y, bias=self.b)])
        self.dx = B.GroupedCall(GROUPED_DX, [B.Group(w=self.W, y_cols=dy, dx_cols=dx)])
        self.dw = B.GroupedCall(GROUPED_DW, [B.Group(w=self.W, x_cols=x, y_cols=dy, dw=self.dW,
                                                     dbias=self.db)])
        self.flops = 3 * 2 * 4 * H * (E + H) * n
        self.units = n
        self.side, self.zeroed = torch.cuda.Stream(), torch.cuda.Event()

    def step(self):
        # The weight gradient runs on a second stream beside the forward and input-gradient
        # launches (as the C++ BatchedGraph schedules it): its CTAs fill the SMs those leave idle
        # in their last wave.
        main = torch.cuda.current_stream()
        self.grads.zero_()
        self.zeroed.record(main)
        self.side.wait_event(self.zeroed)
        self.fwd()
        self.dw.run(self.side.cuda_stream)
        self.dx()
        main.wait_stream(self.side)


class MlpDataParallel:
    """Config 5: Affine+ReLU 784 -> 1024 -> 1024 -> 10, softmax cross-entropy summed over the
    batch, Adam (lr 1e-3, per-element clip 5, eps 1e-8, betas 0.9/0.999: ginn/update/update.h:
    92-133), 4096 columns per rank (the examples/mnist-dp.cu pattern, one process per GPU).
    All gradients live in one flat buffer that is all-reduced once per step; every rank then
    applies the same Adam update, so the replicas stay identical."""

    DIMS = (784, 1024, 1024, 10)

    def __init__(self, device, rank=0, world=1, batch=4096, allreduce=None):
        gw = torch.Generator(device=device).manual_seed(123457)          # same weights everywhere
        gd = torch.Generator(device=device).manual_seed(123457 + 1 + rank)  # own data per rank
        d = self.DIMS
        # flat layout W1 b1 | W2 b2 W3 b3: the gradients of layers 2 and 3 are complete before
        # layer 1's weight gradient starts and form one contiguous bucket for the all-reduce
        sizes = [d[1] * d[0], d[1], d[2] * d[1], d[2], d[3] * d[2], d[3]]
        total = sum(sizes)
        self.params = torch.empty(total, device=device)
        self.grads = torch.zeros(total, device=device)
        self.m = torch.zeros(total, device=device)
        self.v = torch.zeros(total, device=device)
        views, gviews, off = [], [], 0
        for n in sizes:
            views.append(self.params[off:off + n])
            gviews.append(self.grads[off:off + n])
            off += n
        self.bucket_late = self.grads[:sizes[0] + sizes[1]]    # layer 1: ready last
        self.bucket_early = self.grads[sizes[0] + sizes[1]:]   # layers 2 and 3
        cmv = lambda flat, r, c: torch.as_strided(flat, (r, c), (1, r))
        self.W = [cmv(views[2 * i], d[i + 1], d[i]) for i in range(3)]
        self.dW = [cmv(gviews[2 * i], d[i + 1], d[i]) for i in range(3)]
        self.b, self.db = [views[2 * i + 1] for i in range(3)], [gviews[2 * i + 1] for i in range(3)]
        for i in range(3):
            self.W[i].copy_(_xavier(d[i + 1], d[i], gw, device))
            self.b[i].copy_(_xavier(d[i + 1], 1, gw, device).reshape(-1))
        self.x = B.colmajor(d[0], batch, torch.float32, device)
        self.x.copy_(torch.rand(d[0], batch, device=device, generator=gd))
        self.labels = torch.randint(0, 10, (batch,), device=device, generator=gd)
        self.labels32 = self.labels.to(torch.int32)
        self.smax = B.colmajor(d[3], batch, torch.float32, device, fill=0.0)
        self.nll = torch.zeros(batch, device=device)
        self.ones = torch.ones(batch, device=device)  # d(sum of the losses) / d(each loss)
        self.h = [self.x] + [B.colmajor(d[i + 1], batch, torch.float32, device, fill=0.0) for i in range(3)]
        # the three activation gradients in one buffer: one fill per step
        self.dh_flat = torch.zeros(sum(d[1:]) * batch, device=device)
        offs = [0, d[1] * batch, (d[1] + d[2]) * batch]
        self.dh = [None] + [torch.as_strided(self.dh_flat, (d[i + 1], batch), (1, d[i + 1]), offs[i])
                            for i in range(3)]
        self.acts = (B.ACT_RELU, B.ACT_RELU, B.ACT_NONE)
        self.allreduce, self.world, self.batch, self.t = allreduce, world, batch, 0
        self.loss = torch.zeros((), device=device)
        fwd = sum(2 * d[i + 1] * d[i] * batch for i in range(3))
        self.flops = 2 * fwd + sum(2 * d[i + 1] * d[i] * batch for i in (1, 2))  # fwd + dW + dX(2,3)
        self.units = batch

    def _front(self):
        """reset_grad, forward, loss, backward of layers 3 and 2 (everything before the first
        all-reduce can start)."""
        gb = B
        self.grads.zero_()
        self.dh_flat.zero_()
        for i in range(3):
            gb.affine_forward([gb.Pair(self.W[i], self.h[i])], self.b[i], self.acts[i], self.h[i + 1])
        # loss = Sum(PickNegLogSoftmax(logits, labels)) (examples/mnist-dp.cu:141) and its gradient
        gb.pick_nll_forward(self.h[3], self.labels32, self.smax, self.nll)
        self.loss = self.nll.sum()
        gb.pick_nll_backward(self.smax, self.labels32, self.ones, self.dh[3])
        for i in (2, 1):
            self._backward_layer(i)

    def _backward_layer(self, i):
        B.affine_backward([B.PairGrad(self.W[i], self.h[i], self.dW[i],
                                      self.dh[i] if i > 0 else None)],
                          self.dh[i + 1], self.h[i + 1], self.acts[i], self.db[i])

    def _back(self):
        self._backward_layer(0)

    def capture(self):
        """Records the two launch sequences of a step (before the first all-reduce; layer 1's
        backward) into CUDA graphs; the collectives and Adam (whose step count is a host scalar)
        stay ordinary calls.  With eight processes on one host the ~25 launches of a step
        otherwise take the host about as long as they take the GPU."""
        self._graphs = (graphed(self._front), graphed(self._back))

    def step(self):
        gb = B
        front, back = getattr(self, "_graphs", None) or (self._front, self._back)
        front()
        wait = []
        # data parallel: the all-reduce of layers 2 and 3 runs beside layer 1's backward
        # product; `allreduce` returns a function that makes this stream wait for the result
        if self.allreduce is not None and self.world > 1:
            wait.append(self.allreduce(self.bucket_early))
        back()
        if self.allreduce is not None and self.world > 1:
            wait.append(self.allreduce(self.bucket_late))
            for w in wait:
                w()
        # Adam on the flat buffers (ginn/update/update.h:115-133), one kernel
        self.t += 1
        gb.adam_update(self.params, self.grads, self.m, self.v, self.t)
