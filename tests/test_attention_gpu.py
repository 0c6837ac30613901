"""GPU parity of the attention entry points against the oracle (fp64 restatement of min-GPT's
BatchedProd -> scale -> mask -> Softmax -> BatchedProd, examples/min-gpt.cu.cpp:124-157): the
one-kernel forward at several shapes with and without scale / causal mask / kept softmax output,
the unfused sequence the library takes for other shapes, the composed backward, and the full
config-3 size against the separate BatchedProd + Softmax calls."""
import os

import numpy as np
import pytest
import torch

from oracle import oracle as orc
from ginn_b200 import binding as B
from helpers import check, randn

pytestmark = pytest.mark.gpu


def make(rng, T, hs, nb, dt=np.float32):
    s = np.sqrt(1 / 8)
    return randn(rng, (T, hs, nb), dt, s), randn(rng, (hs, T, nb), dt, s), randn(rng, (hs, T, nb), dt, s)


@pytest.mark.parametrize("T,hs,nb", [(256, 64, 4), (128, 64, 3), (256, 32, 2), (256, 128, 2),
                                      (192, 64, 2), (64, 32, 5), (36, 32, 2)])
@pytest.mark.parametrize("scale,causal", [(1.0, False), (0.125, True)])
def test_fused_forward(gpu, T, hs, nb, scale, causal):
    if os.environ.get("GINN_B200_TEST_PATH", "0") != "0":
        pytest.skip("the fused kernel serves the automatic path only; a forced path composes the pass")
    rng = np.random.default_rng(71)
    k, q, v = make(rng, T, hs, nb)
    kd, qd, vd = map(B.from_host, (k, q, v))
    o = B.colmajor(hs, T, torch.float32, batches=nb, fill=7.0)
    p = B.colmajor(T, T, torch.float32, batches=nb, fill=7.0)
    launches = gpu.launch_count()
    gpu.attention_forward(kd, qd, vd, o, p, scale, causal)
    torch.cuda.synchronize()
    assert gpu.launch_count() == launches + 1            # one kernel
    ro, rp = orc.attention_forward(k, q, v, scale, causal)
    check(B.to_host(p), rp, np.float32, "softmax output")
    check(B.to_host(o), ro, np.float32, "attention output")
    if causal:
        assert (B.to_host(p)[np.triu_indices(T, 1)[::-1]] == 0).all()   # keys after the query
    o2 = B.colmajor(hs, T, torch.float32, batches=nb, fill=7.0)
    gpu.attention_forward(kd, qd, vd, o2, None, scale, causal)           # softmax output not kept
    torch.cuda.synchronize()
    check(B.to_host(o2), ro, np.float32, "attention output, p not kept")


def test_unfused_sequence_for_other_shapes(gpu):
    """T above the one-kernel limit, and Half: the library runs the reference's sequence with p
    as the score buffer."""
    rng = np.random.default_rng(72)
    k, q, v = make(rng, 320, 48, 2)
    o = B.colmajor(48, 320, torch.float32, batches=2, fill=0.0)
    p = B.colmajor(320, 320, torch.float32, batches=2, fill=0.0)
    gpu.attention_forward(*map(B.from_host, (k, q, v)), o, p, 0.25, True)
    torch.cuda.synchronize()
    ro, rp = orc.attention_forward(k, q, v, 0.25, True)
    check(B.to_host(p), rp, np.float32)
    check(B.to_host(o), ro, np.float32)
    with pytest.raises(gpu.GinnB200Error):
        gpu.attention_forward(*map(B.from_host, (k, q, v)), o, None)      # no score buffer
    kh, qh, vh = make(rng, 128, 64, 2, np.float16)
    oh = B.colmajor(64, 128, torch.float16, batches=2, fill=0.0)
    ph = B.colmajor(128, 128, torch.float16, batches=2, fill=0.0)
    gpu.attention_forward(*map(B.from_host, (kh, qh, vh)), oh, ph)
    torch.cuda.synchronize()
    ro, rp = orc.attention_forward(kh, qh, vh)
    check(B.to_host(oh), ro, np.float16)


@pytest.mark.parametrize("scale,causal", [(1.0, False), (0.125, True)])
def test_backward(gpu, scale, causal):
    rng = np.random.default_rng(73)
    T, hs, nb = 256, 64, 3
    k, q, v = make(rng, T, hs, nb)
    d_o = randn(rng, (hs, T, nb), np.float32)
    kd, qd, vd, dod = map(B.from_host, (k, q, v, d_o))
    o = B.colmajor(hs, T, torch.float32, batches=nb, fill=0.0)
    p = B.colmajor(T, T, torch.float32, batches=nb, fill=0.0)
    ds = B.colmajor(T, T, torch.float32, batches=nb, fill=0.0)
    gpu.attention_forward(kd, qd, vd, o, p, scale, causal)
    dk = B.colmajor(T, hs, torch.float32, batches=nb, fill=0.5)
    dq = B.colmajor(hs, T, torch.float32, batches=nb, fill=0.5)
    dv = B.colmajor(hs, T, torch.float32, batches=nb, fill=0.5)
    gpu.attention_backward(kd, qd, vd, p, dod, ds, dk, dq, dv, scale)
    torch.cuda.synchronize()
    rdk, rdq, rdv = orc.attention_backward(k, q, v, B.to_host(p), d_o, scale)
    check(B.to_host(dk), 0.5 + rdk.astype(np.float64), np.float32, "dk +=")
    check(B.to_host(dq), 0.5 + rdq.astype(np.float64), np.float32, "dq +=")
    check(B.to_host(dv), 0.5 + rdv.astype(np.float64), np.float32, "dv +=")


def test_config3_fused_equals_separate_calls(gpu):
    """Full config 3 (256 batches, T = 256, hs = 64): the fused step against the BatchedProd +
    Softmax sequence of the benchmark harness, and both against the oracle on a few batches."""
    from ginn_b200.workloads import Attention
    dev = torch.device("cuda", 0)
    a, b = Attention(dev, fused=True), Attention(dev, fused=False)
    a.step()
    b.step()
    torch.cuda.synchronize()
    for name in ("O", "P", "dK", "dQ", "dV"):
        x, y = getattr(a, name).double(), getattr(b, name).double()
        assert float((x - y).norm() / y.norm()) <= 1e-5, name
    sel = [0, 101, 255]
    host = lambda t: t[:, :, sel].cpu().numpy()
    ro, rp = orc.attention_forward(host(a.k), host(a.q), host(a.v))
    check(host(a.O), ro, np.float32, "O")
    check(host(a.P), rp, np.float32, "P")


def test_backward_on_one_stream_in_a_graph_and_with_missing_gradients(gpu):
    """The backward entry forks dV and dQ onto a second stream and joins it again inside the
    call.  The same pass with the option off, recorded into a CUDA graph (the fork must join the
    capture) and with some gradients not asked for must agree with the default."""
    rng = np.random.default_rng(74)
    T, hs, nb = 256, 64, 5
    k, q, v = make(rng, T, hs, nb)
    d_o = randn(rng, (hs, T, nb), np.float32)
    kd, qd, vd, dod = map(B.from_host, (k, q, v, d_o))
    o = B.colmajor(hs, T, torch.float32, batches=nb, fill=0.0)
    p = B.colmajor(T, T, torch.float32, batches=nb, fill=0.0)
    gpu.attention_forward(kd, qd, vd, o, p)
    z = lambda r, c: B.colmajor(r, c, torch.float32, batches=nb, fill=0.0)

    def run(dk=True, dq=True, dv=True):
        ds = z(T, T)
        out = (z(T, hs) if dk else None, z(hs, T) if dq else None, z(hs, T) if dv else None)
        gpu.attention_backward(kd, qd, vd, p, dod, ds, *out)
        torch.cuda.synchronize()
        return out

    ref = run()
    rdk, rdq, rdv = orc.attention_backward(k, q, v, B.to_host(p), d_o, 1.0)
    for got, want, name in zip(ref, (rdk, rdq, rdv), ("dk", "dq", "dv")):
        check(B.to_host(got), want, np.float32, name)
    # not bit for bit: with this few tiles the contraction is split over CTAs that add their
    # parts in the order they finish
    close = lambda x, y: float((x.double() - y.double()).norm() / y.double().norm()) <= 2e-6
    same = lambda a, b: all(x is None or close(x, y) for x, y in zip(a, b))
    try:
        gpu.set_option("fork_streams", 0)
        assert same(run(), ref)
    finally:
        gpu.set_option("fork_streams", 1)
    assert same(run(dk=False), ref)
    assert same(run(dq=False), ref)
    assert same(run(dk=False, dq=False), ref)
    # recorded into a graph and replayed twice: gradients accumulate
    ds = z(T, T)
    out = (z(T, hs), z(hs, T), z(hs, T))
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        gpu.attention_backward(kd, qd, vd, p, dod, ds, *out)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    for t in out:
        t.zero_()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        gpu.attention_backward(kd, qd, vd, p, dod, ds, *out)
    g.replay()
    g.replay()
    torch.cuda.synchronize()
    for got, want, name in zip(out, ref, ("dk", "dq", "dv")):
        assert float((got.double() - 2 * want.double()).norm() / want.double().norm()) <= 2e-6, name
