"""GPU parity of the fused Affine forward/backward entry points against the oracle."""
import numpy as np
import pytest
import torch

from oracle import oracle as orc
from ginn_b200 import binding as B
from helpers import check, check_elementwise, randn

pytestmark = pytest.mark.gpu
ACTS = [orc.ACT_NONE, orc.ACT_TANH, orc.ACT_SIGMOID, orc.ACT_RELU]


def zeros_like_cm(x):
    return B.colmajor(x.shape[0], x.shape[1], x.dtype, fill=0.0)


def test_known_answers(gpu, kat):
    """test/nodes.cu.cpp:1117-1196 (Affine, AffineSigmoid, broadcast, high rank)."""
    for dt, eps in [(np.float32, 2e-6), (np.float16, kat["eps"]["f16_affine"])]:
        a = kat["affine"]
        W, V, b = (B.from_host(np.asarray(a[k], dt)) for k in ("W", "V", "b"))
        out = B.colmajor(2, 1, W.dtype, fill=0.0)
        gpu.affine_forward([gpu.Pair(W, V)], b, gpu.ACT_NONE, out)
        torch.cuda.synchronize()
        np.testing.assert_allclose(B.to_host(out), np.asarray(a["WVb"]), rtol=eps)
        gpu.affine_forward([gpu.Pair(W, V)], b, gpu.ACT_SIGMOID, out)
        torch.cuda.synchronize()
        np.testing.assert_allclose(B.to_host(out), np.asarray(a["sigmoid"]), rtol=eps)
        bc = kat["affine_broadcast"]
        W, V, b = (B.from_host(np.asarray(bc[k], dt)) for k in ("W", "V", "b"))
        out = B.colmajor(2, 2, W.dtype, fill=0.0)
        gpu.affine_forward([gpu.Pair(W, V)], b, gpu.ACT_NONE, out)
        torch.cuda.synchronize()
        np.testing.assert_allclose(B.to_host(out), np.asarray(bc["WVb"]), rtol=eps)
        h = kat["affine_high_rank"]
        V3 = np.asarray(h["V"], dt)
        V2 = V3.reshape(orc.fold2(V3.shape), order="F")
        out = B.colmajor(2, 4, W.dtype, fill=0.0)
        gpu.affine_forward([gpu.Pair(W, B.from_host(V2))], B.from_host(np.asarray(h["b"], dt)),
                           gpu.ACT_NONE, out)
        torch.cuda.synchronize()
        np.testing.assert_allclose(B.to_host(out).reshape(h["WVb_shape"], order="F"),
                                   np.asarray(h["WVb"]), rtol=eps)


def test_lstm_golden_through_fused_affines(gpu):
    """test/model.cpp:22-66 with every gate computed by ginn_b200_affine_forward."""
    f32 = np.float32
    Wm = B.from_host(np.asarray([[0.0, 0.1, 0.2], [0.3, 0.4, 0.5], [0.6, 0.7, -1.1]], f32))
    Z = B.from_host(np.zeros((3, 3), f32))
    b = B.from_host(np.asarray([0.0, 0.3, 0.6], f32))
    h = B.from_host(np.asarray([[0.3], [0.5], [0.7]], f32))
    c = B.from_host(np.asarray([[-0.3], [-0.5], [-0.7]], f32))
    x = B.from_host(np.asarray([[0.25], [-0.5], [0.75]], f32))

    def aff(act, *pairs):
        out = B.colmajor(3, 1, torch.float32, fill=0.0)
        gpu.affine_forward([gpu.Pair(a_, b_) for a_, b_ in pairs], b, act, out)
        return out
    for _ in range(5):
        i = aff(gpu.ACT_SIGMOID, (Wm, x), (Wm, h), (Z, c))
        f = aff(gpu.ACT_SIGMOID, (Wm, x), (Wm, h), (Z, c))
        g = aff(gpu.ACT_TANH, (Wm, x), (Wm, h))
        c = f * c + i * g
        o = aff(gpu.ACT_SIGMOID, (Wm, x), (Wm, h), (Z, c))
        h = o * torch.tanh(c)
    torch.cuda.synchronize()
    np.testing.assert_allclose(B.to_host(h).ravel(), [0.067673, 0.504593, -0.030797], rtol=2e-5)
    np.testing.assert_allclose(B.to_host(c).ravel(), [0.127502, 0.972858, -0.062305], rtol=2e-5)


@pytest.mark.parametrize("dt", [np.float32, np.float16])
@pytest.mark.parametrize("act", ACTS)
def test_forward_backward_config1_shape(gpu, dt, act):
    """Config 1 (W 512x784, X 784x128, tanh) plus a second pair, all fused nonlinearities.
    Backward runs twice into the same gradients: the reference's e+e accumulation check."""
    rng = np.random.default_rng(21 + act)
    m, n, k1, k2 = 512, 128, 784, 100
    a_x = np.sqrt(6 / (0.5 * (m + k1)))
    W = rng.uniform(-a_x, a_x, (m, k1)).astype(dt)
    V = rng.uniform(-a_x, a_x, (m, k2)).astype(dt)
    X, H = randn(rng, (k1, n), dt), randn(rng, (k2, n), dt)
    b = rng.uniform(-a_x, a_x, m).astype(dt)
    dY = randn(rng, (m, n), dt)
    Wd, Vd, Xd, Hd, bd, dYd = map(B.from_host, (W, V, X, H, b, dY))
    Y = B.colmajor(m, n, Wd.dtype, fill=0.0)
    gpu.affine_forward([gpu.Pair(Wd, Xd), gpu.Pair(Vd, Hd)], bd, act, Y)
    torch.cuda.synchronize()
    y = B.to_host(Y)
    check(y, orc.affine_forward([(W, X), (V, H)], b, act), dt, "value")
    dW, dX, dV = zeros_like_cm(Wd), zeros_like_cm(Xd), zeros_like_cm(Vd)
    db = torch.zeros(m, device="cuda", dtype=Wd.dtype)
    for _ in range(2):
        gpu.affine_backward([gpu.PairGrad(Wd, Xd, dW, dX), gpu.PairGrad(Vd, Hd, dV, None)], dYd,
                            Y, act, db)
    torch.cuda.synchronize()
    g = orc.affine_backward([(W, X), (V, H)], dY, y, act, dt)
    if dt == np.float16:  # the second accumulation rounds the running fp16 sum once more
        tw = lambda v: 2 * np.asarray(v)
    else:
        tw = lambda v: 2 * np.asarray(v)
    check(B.to_host(dW), tw(g["da"][0]), dt, "dW")
    check(B.to_host(dX), tw(g["db"][0]), dt, "dX")
    check(B.to_host(dV), tw(g["da"][1]), dt, "dV")
    check(B.to_host(db), tw(g["dbias"]), dt, "db")


@pytest.mark.parametrize("dt", [np.float32, np.float16])
@pytest.mark.parametrize("act", [orc.ACT_NONE, orc.ACT_SIGMOID])
def test_reference_elementwise_rule_on_affine(gpu, dt, act):
    """The reference compares every element of the value and of every gradient between its CPU
    and GPU runs (test/check_node.h:104-119: within eps relatively, or both near zero) on
    well-scaled inputs; the same rule on a two-pair Affine with positive operands, so that no
    element is a difference of large numbers."""
    rng = np.random.default_rng(41 + act)
    m, n, k1, k2 = 130, 70, 96, 40
    pos = lambda shape, s: (np.abs(rng.standard_normal(shape)) * s + 0.1 * s).astype(dt)
    W, V, X, H, b = pos((m, k1), 0.02), pos((m, k2), 0.02), pos((k1, n), 1), pos((k2, n), 1), pos(m, 0.1)
    dY = pos((m, n), 1)
    Wd, Vd, Xd, Hd, bd, dYd = map(B.from_host, (W, V, X, H, b, dY))
    Y = B.colmajor(m, n, Wd.dtype, fill=0.0)
    gpu.affine_forward([gpu.Pair(Wd, Xd), gpu.Pair(Vd, Hd)], bd, act, Y)
    dW, dX, dV, dH = zeros_like_cm(Wd), zeros_like_cm(Xd), zeros_like_cm(Vd), zeros_like_cm(Hd)
    db = torch.zeros(m, device="cuda", dtype=Wd.dtype)
    gpu.affine_backward([gpu.PairGrad(Wd, Xd, dW, dX), gpu.PairGrad(Vd, Hd, dV, dH)], dYd, Y, act, db)
    torch.cuda.synchronize()
    y = B.to_host(Y)
    check_elementwise(y, orc.affine_forward([(W, X), (V, H)], b, act), dt, "value")
    g = orc.affine_backward([(W, X), (V, H)], dY, y, act, dt)
    for got, ref, what in [(dW, g["da"][0], "dW"), (dX, g["db"][0], "dX"), (dV, g["da"][1], "dV"),
                           (dH, g["db"][1], "dH"), (db, g["dbias"], "db")]:
        check_elementwise(B.to_host(got), np.asarray(ref), dt, what)


@pytest.mark.parametrize("act", ACTS)
def test_forward_with_split_contraction(gpu, act):
    """Few output tiles and a long contraction: the fp32 path splits K over several CTAs, adds
    the partial sums (and the bias) atomically into a zeroed output and applies the activation
    in a pass over the summed result.  Config 1's exact shape, one with ragged edge tiles, and
    a padded output; run twice: stale contents of the output must not leak into the sums."""
    rng = np.random.default_rng(51 + act)
    for (m, n, k, pad) in [(512, 128, 784, 0), (130, 70, 1000, 0), (256, 96, 2048, 4)]:
        W, X, b = randn(rng, (m, k), np.float32, 0.05), randn(rng, (k, n), np.float32), randn(rng, m, np.float32)
        Wd, Xd, bd = map(B.from_host, (W, X, b))
        Y = B.colmajor(m, n, torch.float32, ld=m + pad, fill=7.0)   # stale contents must not leak
        ref = orc.affine_forward([(W, X)], b, act)
        for _ in range(2):
            gpu.affine_forward([gpu.Pair(Wd, Xd)], bd, act, Y)
            torch.cuda.synchronize()
            check(B.to_host(Y), ref, np.float32, f"{m}x{n}x{k} act {act}")


@pytest.mark.parametrize("act", ACTS)
def test_half_layers_on_the_tma_kernels(gpu, act):
    """Half Affines large enough for the TMA-fed kernels: bias and nonlinearity run in the
    epilogue of the last pair's product (one and two pairs, ragged edge tiles, an output whose
    leading dimension rules out 16-byte stores); then the backward pass of a layer whose weight
    gradient has few tiles and a long contraction, run twice onto the same gradients."""
    rng = np.random.default_rng(61 + act)
    dt = np.float16
    for (m, n, k1, k2, pad) in [(256, 512, 256, 0, 0), (200, 264, 136, 72, 0), (256, 256, 128, 64, 3)]:
        W, X, b = randn(rng, (m, k1), dt, 0.05), randn(rng, (k1, n), dt), randn(rng, m, dt)
        pairs_h, pairs_d = [(W, X)], [gpu.Pair(B.from_host(W), B.from_host(X))]
        if k2:
            V, H = randn(rng, (m, k2), dt, 0.05), randn(rng, (k2, n), dt)
            pairs_h.append((V, H))
            pairs_d.append(gpu.Pair(B.from_host(V), B.from_host(H)))
        Y = B.colmajor(m, n, torch.float16, ld=m + pad, fill=7.0)
        gpu.affine_forward(pairs_d, B.from_host(b), act, Y)
        torch.cuda.synchronize()
        check(B.to_host(Y), orc.affine_forward(pairs_h, b, act), dt, f"value {m}x{n} pad {pad}")
    m, n, k = 256, 4096, 256
    W, X, b, dY = randn(rng, (m, k), dt, 0.05), randn(rng, (k, n), dt), randn(rng, m, dt), randn(rng, (m, n), dt, 0.1)
    Wd, Xd, bd, dYd = map(B.from_host, (W, X, b, dY))
    Y = B.colmajor(m, n, torch.float16, fill=0.0)
    gpu.affine_forward([gpu.Pair(Wd, Xd)], bd, act, Y)
    dW, dX = zeros_like_cm(Wd), zeros_like_cm(Xd)
    db = torch.zeros(m, device="cuda", dtype=torch.float16)
    for _ in range(2):
        gpu.affine_backward([gpu.PairGrad(Wd, Xd, dW, dX)], dYd, Y, act, db)
    torch.cuda.synchronize()
    g = orc.affine_backward([(W, X)], dY, B.to_host(Y), act, dt)
    check(B.to_host(dW), 2 * np.asarray(g["da"][0]), dt, "dW")
    check(B.to_host(dX), 2 * np.asarray(g["db"][0]), dt, "dX")
    check(B.to_host(db), 2 * np.asarray(g["dbias"]), dt, "db")


def test_half_layer_on_the_cta_pair_kernel(gpu):
    """A Half Affine with at least a wave of 256 x 256 tiles runs on the CTA-pair kernel, which
    applies bias and nonlinearity in its epilogue too (second pair accumulating onto the first)."""
    rng = np.random.default_rng(67)
    dt = np.float16
    m, n, k1, k2 = 2048, 4864, 256, 128
    W, X, b = randn(rng, (m, k1), dt, 0.05), randn(rng, (k1, n), dt), randn(rng, m, dt)
    V, H = randn(rng, (m, k2), dt, 0.05), randn(rng, (k2, n), dt)
    for act in (orc.ACT_TANH, orc.ACT_NONE):
        Y = B.colmajor(m, n, torch.float16, fill=7.0)
        gpu.affine_forward([gpu.Pair(B.from_host(W), B.from_host(X)), gpu.Pair(B.from_host(V), B.from_host(H))],
                           B.from_host(b), act, Y)
        torch.cuda.synchronize()
        check(B.to_host(Y), orc.affine_forward([(W, X), (V, H)], b, act), dt, f"pair kernel act {act}")


def test_half_backward_with_the_nodes_own_scratch(gpu):
    """A large Half Affine with a nonlinearity materialises dY (.) f'(Y) once.  Given the node's
    own d-pre-activation tensor (as AffineNode owns dpreactiv_, ginn/node/affine.h:82) dA stays
    out of the library's pool: same gradients as with the library's stream-ordered scratch, and
    the device's free memory does not move once the pool holds the small partial-sum buffers."""
    rng = np.random.default_rng(55)
    m, n, k = 512, 256, 384
    dt = np.float16
    W, X, b, dY = randn(rng, (m, k), dt, 0.05), randn(rng, (k, n), dt), randn(rng, m, dt), randn(rng, (m, n), dt)
    Wd, Xd, bd, dYd = map(B.from_host, (W, X, b, dY))
    Y = B.colmajor(m, n, torch.float16, fill=0.0)
    gpu.affine_forward([gpu.Pair(Wd, Xd)], bd, gpu.ACT_TANH, Y)
    scratch = B.colmajor(m, n, torch.float16, fill=0.0)
    results = []
    for ws in (None, scratch, scratch):
        dW, dX = zeros_like_cm(Wd), zeros_like_cm(Xd)
        db = torch.zeros(m, device="cuda", dtype=torch.float16)
        torch.cuda.synchronize()
        free0 = torch.cuda.mem_get_info()[0]
        gpu.affine_backward([gpu.PairGrad(Wd, Xd, dW, dX)], dYd, Y, gpu.ACT_TANH, db, ws)
        torch.cuda.synchronize()
        if ws is not None and len(results) == 2:      # second call with the scratch: all warm
            assert torch.cuda.mem_get_info()[0] == free0
        results.append([B.to_host(t) for t in (dW, dX, db)])
    g = orc.affine_backward([(W, X)], dY, B.to_host(Y), orc.ACT_TANH, dt)
    for got in results:
        check(got[0], g["da"][0], dt, "dW")
        check(got[1], g["db"][0], dt, "dX")
        check(got[2], g["dbias"], dt, "db")


def test_bias_gradient_alone(gpu):
    """Only the bias has a gradient (no weight gradient to ride on)."""
    rng = np.random.default_rng(31)
    m, n, k = 70, 33, 20
    W, X, dY = randn(rng, (m, k), np.float32), randn(rng, (k, n), np.float32), randn(rng, (m, n), np.float32)
    Wd, Xd, dYd = map(B.from_host, (W, X, dY))
    Y = B.colmajor(m, n, torch.float32, fill=0.0)
    gpu.affine_forward([gpu.Pair(Wd, Xd)], None, gpu.ACT_SIGMOID, Y)
    db = torch.ones(m, device="cuda")
    gpu.affine_backward([gpu.PairGrad(Wd, Xd, None, None)], dYd, Y, gpu.ACT_SIGMOID, db)
    torch.cuda.synchronize()
    g = orc.affine_backward([(W, X)], dY, B.to_host(Y), orc.ACT_SIGMOID, np.float32)
    check(B.to_host(db), 1 + g["dbias"], np.float32)


def test_mlp_last_layer_rows_of_ten(gpu):
    """Config 5's output layer: W 10x1024, batch 4096 -- leading dimensions of 40 bytes."""
    rng = np.random.default_rng(32)
    m, k, n = 10, 1024, 512
    W, X, b, dY = randn(rng, (m, k), np.float32, 0.05), randn(rng, (k, n), np.float32), \
        randn(rng, m, np.float32), randn(rng, (m, n), np.float32)
    Wd, Xd, bd, dYd = map(B.from_host, (W, X, b, dY))
    Y = B.colmajor(m, n, torch.float32, fill=0.0)
    gpu.affine_forward([gpu.Pair(Wd, Xd)], bd, gpu.ACT_NONE, Y)
    dW, dX, db = zeros_like_cm(Wd), zeros_like_cm(Xd), torch.zeros(m, device="cuda")
    gpu.affine_backward([gpu.PairGrad(Wd, Xd, dW, dX)], dYd, None, gpu.ACT_NONE, db)
    torch.cuda.synchronize()
    check(B.to_host(Y), orc.affine_forward([(W, X)], b, orc.ACT_NONE), np.float32)
    g = orc.affine_backward([(W, X)], dY, None, orc.ACT_NONE, np.float32)
    check(B.to_host(dW), g["da"][0], np.float32)
    check(B.to_host(dX), g["db"][0], np.float32)
    check(B.to_host(db), g["dbias"], np.float32)


def test_affine_argument_errors(gpu):
    x = torch.zeros(64, device="cuda")
    W = torch.as_strided(x, (2, 3), (1, 2))
    with pytest.raises(gpu.GinnB200Error):
        gpu.affine_forward([gpu.Pair(W, W)] * 5, None, gpu.ACT_NONE, W)   # more than 4 pairs
    with pytest.raises(gpu.GinnB200Error):
        gpu.affine_forward([gpu.Pair(W, W)], None, 9, W)                  # unknown activation
