"""CPU-only: the oracle against the reference's known answers, the C port against the oracle,
and the C ABI's symbol table against include/ginn_b200.h."""
import ctypes
import os
import re

import numpy as np
import pytest

from oracle import oracle as orc

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def arr(x, dt=np.float32):
    return np.asarray(x, dtype=dt)


@pytest.mark.parametrize("dt,eps_key", [(np.float32, "f32"), (np.float16, "f16_prod")])
def test_prod_known_answer(kat, dt, eps_key):
    p = kat["prod"]
    out = orc.gemm(arr(p["W"], dt), arr(p["V"], dt)).astype(dt)
    np.testing.assert_allclose(out, arr(p["WV"]), rtol=kat["eps"][eps_key], atol=1e-6)


@pytest.mark.parametrize("dt,eps_key", [(np.float32, "f32"), (np.float16, "f16_affine")])
def test_affine_known_answers(kat, dt, eps_key):
    a = kat["affine"]
    W, V, b = arr(a["W"], dt), arr(a["V"], dt), arr(a["b"], dt)
    eps = kat["eps"][eps_key]
    ident = orc.affine_forward([(W, V)], b, orc.ACT_NONE).astype(dt)
    np.testing.assert_allclose(ident, arr(a["WVb"]), rtol=eps, atol=1e-6)
    sig = orc.affine_forward([(W, V)], b, orc.ACT_SIGMOID).astype(dt)
    np.testing.assert_allclose(sig, arr(a["sigmoid"]), rtol=max(eps, 2e-6), atol=1e-6)
    # Softmax is not fused: the node keeps the pre-activation and runs the reference op after.
    pre = orc.affine_forward([(W, V)], b, orc.ACT_NONE)
    sm = np.exp(pre - pre.max(0)) / np.exp(pre - pre.max(0)).sum(0)
    np.testing.assert_allclose(sm, arr(a["softmax"]), rtol=max(eps, 2e-6))


def test_affine_broadcast_and_high_rank(kat):
    a = kat["affine_broadcast"]
    out = orc.affine_forward([(arr(a["W"]), arr(a["V"]))], arr(a["b"]), orc.ACT_NONE)
    np.testing.assert_allclose(out, arr(a["WVb"]), rtol=1e-6)
    h = kat["affine_high_rank"]
    V = arr(h["V"])                                 # 3 x 2 x 2, column-major in ginn
    rows, cols = orc.fold2(V.shape)
    V2 = V.reshape(rows, cols, order="F")           # rank folded to 2 (ginn/tensor.h:268-282)
    out = orc.affine_forward([(arr(h["W"]), V2)], arr(h["b"]), orc.ACT_NONE)
    np.testing.assert_allclose(out.reshape(h["WVb_shape"], order="F"), arr(h["WVb"]), rtol=1e-6)


def test_pick_nll_known_answer_and_gradient(kat):
    """test/nodes.cu.cpp:755-797: picked softmax and its negative log; the gradient restatement
    against central differences, as the reference's CHECK_ does."""
    k = kat["pick_nll"]
    W, idx = arr(k["W"], np.float64), k["index"]
    smax, val = orc.pick_nll_forward(W, idx)
    np.testing.assert_allclose(smax[idx, np.arange(3)], k["psm"], rtol=1e-6)
    np.testing.assert_allclose(val, k["pnlsm"], rtol=1e-6)
    g = np.array([0.7, -1.3, 2.1])
    dx = orc.pick_nll_backward(smax, idx, g, np.zeros_like(W))
    num = np.zeros_like(W)
    for i in range(W.shape[0]):
        for j in range(W.shape[1]):
            e = np.zeros_like(W)
            e[i, j] = 1e-6
            num[i, j] = ((orc.pick_nll_forward(W + e, idx)[1] - orc.pick_nll_forward(W - e, idx)[1]) * g).sum() / 2e-6
    np.testing.assert_allclose(dx, num, rtol=1e-5, atol=1e-8)


def test_softmax_known_answers_and_gradient(kat):
    """test/nodes.cu.cpp:689-700 for the values; the backward restatement against central
    differences of sum(w * softmax(x))."""
    k = kat["softmax"]
    W = arr(k["W"], np.float64)
    y = orc.pick_nll_forward(W, [0, 0, 0])[0]
    np.testing.assert_allclose(y, k["smaxW"], rtol=1e-6)
    w = np.array([[0.3, -1.0, 2.0], [0.7, 0.2, -0.4]])
    dx = orc.softmax_backward(y, w)
    num = np.zeros_like(W)
    for i in range(2):
        for j in range(3):
            e = np.zeros_like(W)
            e[i, j] = 1e-6
            f = lambda z: (orc.pick_nll_forward(z, [0, 0, 0])[0] * w).sum()
            num[i, j] = (f(W + e) - f(W - e)) / 2e-6
    np.testing.assert_allclose(dx, num, rtol=1e-5, atol=1e-9)


def test_adam_restatement_first_steps():
    """ginn/update/update.h:115-133 by hand: with m = v = 0, step 1 moves every weight by
    -lr * sign(d) (up to eps), whatever the size of d, and clips d in place."""
    w, d = np.array([1.0, -2.0, 0.5]), np.array([0.3, -8.0, 0.0])
    w1, d1, m1, v1 = orc.adam_update(w, d, np.zeros(3), np.zeros(3), 1e-3, 5.0, 1e-8, 0.9, 0.999, 0.9, 0.999)
    np.testing.assert_allclose(d1, [0.3, -5.0, 0.0])
    np.testing.assert_allclose(m1, 0.1 * d1, rtol=1e-6)  # betas are fp32 values, as in the reference
    np.testing.assert_allclose(v1, 0.001 * d1 * d1, rtol=2e-5)
    np.testing.assert_allclose(w1, w - 1e-3 * np.sign(d1), atol=1e-9)


def test_lstm_five_steps_match_recorded_values():
    """test/model.cpp:22-66: five Lstm::step calls (ginn/model/lstm.h:90-105), values recorded
    from PyTorch.  Exercises multi-pair Affines with fused sigmoid/tanh."""
    Wm = arr([[0.0, 0.1, 0.2], [0.3, 0.4, 0.5], [0.6, 0.7, -1.1]])
    Z = np.zeros((3, 3), np.float32)
    b = arr([0.0, 0.3, 0.6])
    h = arr([[0.3], [0.5], [0.7]])
    c = arr([[-0.3], [-0.5], [-0.7]])
    x = arr([[0.25], [-0.5], [0.75]])
    for _ in range(5):
        i = orc.affine_forward([(Wm, x), (Wm, h), (Z, c)], b, orc.ACT_SIGMOID)
        f = orc.affine_forward([(Wm, x), (Wm, h), (Z, c)], b, orc.ACT_SIGMOID)
        g = orc.affine_forward([(Wm, x), (Wm, h)], b, orc.ACT_TANH)
        c = f * c + i * g
        o = orc.affine_forward([(Wm, x), (Wm, h), (Z, c)], b, orc.ACT_SIGMOID)
        h = o * np.tanh(c)
    np.testing.assert_allclose(h.ravel(), [0.067673, 0.504593, -0.030797], rtol=2e-5)
    np.testing.assert_allclose(c.ravel(), [0.127502, 0.972858, -0.062305], rtol=2e-5)


def test_batched_equals_per_slice():
    """test/nodes.cu.cpp:1043-1115: BatchedProd equals per-slice products, rank 3 and rank 4."""
    rng = np.random.default_rng(0)
    a = rng.uniform(-1, 1, (2, 3, 4)).astype(np.float32) + 1
    b = rng.uniform(-1, 1, (3, 5, 4)).astype(np.float32) - 1
    c = orc.gemm_batched(a, b)
    for i in range(4):
        np.testing.assert_allclose(c[:, :, i], a[:, :, i].astype(np.float64) @ b[:, :, i])
    assert orc.fold3((2, 3, 2, 2)) == (2, 3, 4)


def test_backward_matches_finite_differences():
    """The gradient formulas of affine_backward against central differences (the reference's
    check_grad, test/testutil.h:134-171), in fp64."""
    rng = np.random.default_rng(1)
    W, X, V, H = (rng.standard_normal(s) for s in [(4, 3), (3, 5), (4, 2), (2, 5)])
    b = rng.standard_normal(4)
    dout = rng.standard_normal((4, 5))
    for act in (orc.ACT_NONE, orc.ACT_TANH, orc.ACT_SIGMOID):
        out = orc.affine_forward([(W, X), (V, H)], b, act)
        g = orc.affine_backward([(W, X), (V, H)], dout, out, act, np.float64)

        def loss(Wp):
            return float((orc.affine_forward([(Wp, X), (V, H)], b, act) * dout).sum())
        num = np.zeros_like(W)
        for idx in np.ndindex(*W.shape):
            d = np.zeros_like(W)
            d[idx] = 1e-5
            num[idx] = (loss(W + d) - loss(W - d)) / 2e-5
        np.testing.assert_allclose(g["da"][0], num, rtol=1e-6, atol=1e-8)
        np.testing.assert_allclose(g["dbias"], orc.act_backward(out, dout, act).sum(1))


@pytest.mark.parametrize("dt,tol", [(np.float32, 2e-6), (np.float16, 1e-3)])
def test_c_port_matches_oracle(dt, tol):
    rng = np.random.default_rng(2)
    for (m, n, k) in [(1, 1, 1), (5, 7, 3), (33, 65, 129), (300, 70, 257)]:
        for ta in (False, True):
            for tb in (False, True):
                a = rng.standard_normal((k, m) if ta else (m, k)).astype(dt)
                b = rng.standard_normal((n, k) if tb else (k, n)).astype(dt)
                c = rng.standard_normal((m, n)).astype(dt)
                got = orc.cpu_gemm(a, b, ta, tb, c, True, threads=2)
                assert orc.rel_frobenius(got, orc.gemm(a, b, ta, tb, c, True)) < tol


def test_c_port_known_answer(kat):
    p = kat["prod"]
    got = orc.cpu_gemm(arr(p["W"]), arr(p["V"]))
    np.testing.assert_allclose(got, arr(p["WV"]), rtol=1e-6)


def test_library_exports_every_declared_symbol():
    """The C ABI loads without a GPU and exports exactly what include/ginn_b200.h declares."""
    header = open(os.path.join(ROOT, "include", "ginn_b200.h")).read()
    declared = set(re.findall(r"\b(ginn_b200_[a-z_0-9]+)\s*\(", header))
    assert {"ginn_b200_gemm", "ginn_b200_gemm_batched", "ginn_b200_affine_forward",
            "ginn_b200_affine_backward", "ginn_b200_grouped"} <= declared
    import ginn_b200
    lib = ctypes.CDLL(ginn_b200.lib_path())
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared but not exported"
    assert lib.ginn_b200_version() >= 100


def test_bad_option_is_rejected_without_a_gpu():
    import ginn_b200
    with pytest.raises(ginn_b200.GinnB200Error):
        ginn_b200.set_option("no_such_option", 1)


def test_conv2d_known_answers_and_gradients(kat):
    """test/convnodes.cu.cpp:38-109: the reference's Conv2d values (SAME padding, strides), and
    the oracle's gradients against finite differences (the reference checks them the same way)."""
    for case in kat["conv2d"]["cases"]:
        x = np.asarray(case["x"], np.float32)[None, :, :, None]
        f = np.asarray(case["f"], np.float32)[None, None]
        y = orc.conv2d_forward(x, f, *case["strides"])
        np.testing.assert_allclose(y[0, :, :, 0], np.asarray(case["y"], np.float32), rtol=1e-6)
    rng = np.random.default_rng(5)
    for (C, R, W, B, F, KR, KC, sr, sc) in [(3, 5, 6, 2, 4, 3, 2, 2, 1), (2, 7, 4, 1, 3, 2, 3, 1, 3)]:
        x, k = rng.standard_normal((C, R, W, B)), rng.standard_normal((F, C, KR, KC))
        y = orc.conv2d_forward(x, k, sr, sc)
        dy = rng.standard_normal(y.shape)
        dx, dk = orc.conv2d_backward(x, k, dy, sr, sc)
        eps = 1e-6
        for _ in range(5):
            i = tuple(rng.integers(0, s) for s in x.shape)
            xp = x.copy()
            xp[i] += eps
            num = ((orc.conv2d_forward(xp, k, sr, sc) - y) * dy).sum() / eps
            assert abs(num - dx[i]) <= 1e-4 * max(1.0, abs(dx[i]))
            j = tuple(rng.integers(0, s) for s in k.shape)
            kp = k.copy()
            kp[j] += eps
            num = ((orc.conv2d_forward(x, kp, sr, sc) - y) * dy).sum() / eps
            assert abs(num - dk[j]) <= 1e-4 * max(1.0, abs(dk[j]))
