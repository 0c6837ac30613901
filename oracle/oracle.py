"""TEST INFRASTRUCTURE -- not part of the product.  parity: pinned (see below).

fp64 oracle for ginn's dense-contraction path, restated from the reference's CPU branches, and
a ctypes wrapper of the C restatement in cpu_path.c (the reference's own fp32 arithmetic, also
the timed CPU baseline).  Only tests/, bench.py's CPU legs and the smoke check may import this.

Reference lines followed (paths inside the ginn source tree):
  gemm / gemm_batched    ginn/node/prod.h:30-32,41-47,108-117,129-147; shapes and transposes as
                         derived by internal::gpu_prod / gpu_batched_prod (ginn/prod.h:211-310)
  rank folding           ginn/tensor.h:268-282 (trailing dims multiplied into the columns)
  act_forward/backward   ginn/nonlin.h:67-155 (Identity, Tanh, Relu, Sigmoid)
  affine_forward         ginn/node/affine.h:35-77
  affine_backward        ginn/node/affine.h:79-129
  autobatch semantics    ginn/autobatch.h:80-183: a merged product equals the per-node products
  pick_nll_forward       ginn/node/pick.h:60-84,177-182,209-216 with SoftmaxOp::forward,
                         ginn/nonlin.h:162-168
  softmax_backward       ginn/nonlin.h:169-190
  pick_nll_backward      ginn/node/pick.h:87-131,218-224
  lstm_cell_*            ginn/model/lstm.h:97-100 (the elementwise part of the cell)
  adam_update            ginn/update/update.h:92-133
  attention_*            examples/min-gpt.cu.cpp:108-157 (BatchedProd, InPlaceProdScalar,
                         InPlaceMask with an upper-triangular mask, Softmax, BatchedProd) and the
                         backward passes of those nodes (ginn/node/prod.h:129-169, nonlin.h:169-190)
  conv2d_*               ginn/node/conv.h:28-79 over ginn/eigenop/eigen_conv.h:28-190 (patches
                         with Eigen's PADDING_SAME, contraction with the reshaped filters)

Arithmetic: inputs exactly as handed to the GPU (fp32, or fp16-rounded), every product and sum
in fp64, one rounding to the storage type where the reference materialises a tensor (node
value, dpreactiv_, gradients).  The dense product itself lives in Eigen (libeigen/eigen pinned
at 87300c93 by the reference's subprojects/eigen.wrap), which is not vendored with the reference;
its published definition (C_ij = sum_p A_ip B_pj) is what is restated.  Pinning: the known-answer
values of the reference's own tests (test/nodes.cu.cpp:1023-1200, ginn-py/test/test_nodes.py:
804-936) are committed under tests/golden/ and checked by tests/test_oracle.py.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from typing import Optional, Sequence

import numpy as np

ACT_NONE, ACT_TANH, ACT_SIGMOID, ACT_RELU = 0, 1, 2, 3
_HERE = os.path.dirname(os.path.abspath(__file__))


def f64(x) -> np.ndarray:
    return np.asarray(x, dtype=np.float64)


def fold2(shape: Sequence[int]) -> tuple:
    """rows/cols of a ginn tensor: rank folded to 2 (ginn/tensor.h:268-282)."""
    s = list(shape)
    if len(s) == 0:
        return (1, 1)
    if len(s) == 1:
        return (s[0], 1)
    return (s[0], int(np.prod(s[1:])))


def fold3(shape: Sequence[int]) -> tuple:
    s = list(shape) + [1] * (3 - len(shape))
    return (s[0], s[1], int(np.prod(s[2:])))


def gemm(a, b, trans_a=False, trans_b=False, c=None, accumulate=False) -> np.ndarray:
    """fp64 result of op(a) @ op(b) (+ c)."""
    A = f64(a).T if trans_a else f64(a)
    B = f64(b).T if trans_b else f64(b)
    assert A.shape[1] == B.shape[0], "inner dimensions differ (GINN_ASSERT in gpu_prod)"
    out = A @ B
    if accumulate:
        out = out + f64(c)
    return out


def gemm_batched(a, b, trans_a=False, trans_b=False, c=None, accumulate=False) -> np.ndarray:
    """(rows, cols, batch) operands; serial loop over the batch like the reference."""
    batches = a.shape[2]
    outs = [gemm(a[:, :, i], b[:, :, i], trans_a, trans_b,
                 None if c is None else c[:, :, i], accumulate) for i in range(batches)]
    return np.stack(outs, axis=2)


def act_forward(x, act: int, half: bool = False) -> np.ndarray:
    x = f64(x)
    if act == ACT_TANH:
        return np.tanh(x)
    if act == ACT_RELU:
        return np.maximum(x, 0.0)
    if act == ACT_SIGMOID:
        # fp32: 0.5*tanh(0.5x)+0.5; Half: sign-split exponential.  Both equal the logistic function.
        return 0.5 * np.tanh(0.5 * x) + 0.5
    return x


def act_backward(y, dy, act: int) -> np.ndarray:
    y, dy = f64(y), f64(dy)
    if act == ACT_TANH:
        return (1.0 - y * y) * dy
    if act == ACT_RELU:
        return dy * (y > 0)
    if act == ACT_SIGMOID:
        return y * (1.0 - y) * dy
    return dy


def affine_forward(pairs, bias, act: int) -> np.ndarray:
    """fp64 value of act(sum_i a_i @ b_i + bias[:, None])."""
    acc = None
    for a, b in pairs:
        t = f64(a) @ f64(b)
        acc = t if acc is None else acc + t
    if bias is not None:
        acc = acc + f64(bias).reshape(-1, 1)
    return act_forward(acc, act)


def affine_backward(pairs, dout, out, act: int, store_dtype) -> dict:
    """Gradient contributions (fp64) of AffineNode::backward_.

    `store_dtype` is the tensor scalar type: dA = dout (.) act'(out) is rounded to it once, as the
    reference materialises it in dpreactiv_ before the products.
    """
    dA = act_backward(out, dout, act) if act != ACT_NONE else f64(dout)
    dA = f64(dA.astype(store_dtype))
    res = {"dbias": dA.sum(axis=1), "da": [], "db": []}
    for a, b in pairs:
        res["db"].append(f64(a).T @ dA)
        res["da"].append(dA @ f64(b).T)
    return res


def pick_nll_forward(x, index):
    """(smax, value): column softmax of x and -log of the entry index[j] of column j (fp64)."""
    x = f64(x)
    t = np.exp(x - x.max(axis=0, keepdims=True))
    smax = t / t.sum(axis=0, keepdims=True)
    idx = np.asarray(index, dtype=np.int64)
    return smax, -np.log(smax[idx, np.arange(x.shape[1])])


def softmax_backward(y, dy, dx=None):
    """SoftmaxOp::backward (ginn/nonlin.h:169-190): y * (dy - colsum(y * dy)) [+ dx]  (fp64)."""
    y, dy = f64(y), f64(dy)
    out = y * (dy - (y * dy).sum(axis=0, keepdims=True))
    return out if dx is None else f64(dx) + out


def pick_nll_backward(smax, index, grad, dx):
    """dx + (smax - onehot(index)) * grad[None, :]  (fp64)."""
    smax, g = f64(smax), f64(grad).reshape(1, -1)
    out = f64(dx) + smax * g
    idx = np.asarray(index, dtype=np.int64)
    out[idx, np.arange(smax.shape[1])] -= g.ravel()
    return out


def lstm_cell_forward(gates, c_prev):
    """Cell update from one level's merged gate pre-activations (rows i | f | g | o), fp64:
    the composition of ginn/model/lstm.h:97-100.  Returns (activated gates, c, h)."""
    G = f64(gates)
    H = G.shape[0] // 4
    sig = lambda x: 0.5 * np.tanh(0.5 * x) + 0.5
    i, f, g, o = sig(G[:H]), sig(G[H:2 * H]), np.tanh(G[2 * H:3 * H]), sig(G[3 * H:])
    cp = np.zeros_like(i) if c_prev is None else f64(c_prev)[:, :G.shape[1]]
    c = f * cp + i * g
    return np.concatenate([i, f, g, o], 0), c, o * np.tanh(c)


def lstm_cell_backward(act, c, c_prev, dh_next, dc_next, n_next, dh_end=1.0):
    """Gradients of the same update: returns (dgates, dc carried to the previous level)."""
    A, c = f64(act), f64(c)
    H, n = c.shape
    i, f, g, o = A[:H], A[H:2 * H], A[2 * H:3 * H], A[3 * H:]
    cp = np.zeros_like(c) if c_prev is None else f64(c_prev)[:, :n]
    dh = np.full((H, n), float(dh_end))
    dc = np.zeros((H, n))
    if n_next:
        dh[:, :n_next] = f64(dh_next)[:, :n_next]
        dc[:, :n_next] = f64(dc_next)[:, :n_next]
    tc = np.tanh(c)
    dc = dc + dh * o * (1 - tc * tc)
    dG = np.concatenate([dc * g * i * (1 - i), dc * cp * f * (1 - f), dc * i * (1 - g * g),
                         dh * tc * o * (1 - o)], 0)
    return dG, dc * f


def adam_update(w, d, m, v, lr, clip, eps, beta1, beta2, beta1_t, beta2_t):
    """One Adam step (fp64): returns (w, clipped d, m, v); beta*_t are beta^t for this step.
    The hyper-parameters are the reference's `Real` members (ginn/update/update.h:92-97), i.e.
    fp32 values: 1 - beta2 is 0.00099998713, not 0.001."""
    lr, eps, beta1, beta2, beta1_t, beta2_t = (float(np.float32(x)) for x in
                                               (lr, eps, beta1, beta2, beta1_t, beta2_t))
    w, d, m, v = f64(w), f64(d), f64(m), f64(v)
    d = np.clip(d, -clip, clip)
    m = beta1 * m + (1.0 - beta1) * d
    v = beta2 * v + (1.0 - beta2) * d * d
    w = w + (-lr / (1.0 - beta1_t)) * m / (eps + np.sqrt(v / (1.0 - beta2_t)))
    return w, d, m, v


def attention_forward(k, q, v, scale=1.0, causal=False):
    """k (T, hs, nb), q and v (hs, T, nb) -> (o (hs, T, nb), p (T, T, nb)): per batch
    S = scale * k @ q, keys after the query masked to -inf when causal, P = softmax over the
    rows, O = v @ P.  Sums in fp64, one rounding of each returned tensor to the input type."""
    k64, q64, v64 = f64(k), f64(q), f64(v)
    T = k64.shape[0]
    s = scale * np.einsum("ihb,hjb->ijb", k64, q64)
    if causal:
        i, j = np.arange(T)[:, None], np.arange(T)[None, :]
        s = np.where((i > j)[:, :, None], -np.inf, s)
    e = np.exp(s - s.max(axis=0, keepdims=True))
    p = e / e.sum(axis=0, keepdims=True)
    o = np.einsum("hib,ijb->hjb", v64, p)
    dt = np.asarray(k).dtype
    return o.astype(dt), p.astype(dt)


def attention_backward(k, q, v, p, d_o, scale=1.0):
    """(dk, dq, dv) for upstream gradient d_o (hs, T, nb), from the kept softmax output p."""
    k64, q64, v64, p64, do64 = f64(k), f64(q), f64(v), f64(p), f64(d_o)
    dv = np.einsum("hjb,ijb->hib", do64, p64)
    dp = np.einsum("hib,hjb->ijb", v64, do64)
    ds = scale * p64 * (dp - (p64 * dp).sum(axis=0, keepdims=True))
    dk = np.einsum("ijb,hjb->ihb", ds, q64)
    dq = np.einsum("ihb,ijb->hjb", k64, ds)
    dt = np.asarray(k).dtype
    return dk.astype(dt), dq.astype(dt), dv.astype(dt)


def conv2d_geometry(rows, cols, krows, kcols, row_stride, col_stride):
    """Output extents and leading padding of Eigen's PADDING_SAME (eigen_conv.h:40-47 and the
    patch extraction it calls): out = ceil(in / stride), total padding max(0, (out - 1) stride
    + k - in), the smaller half in front."""
    orows, ocols = -(-rows // row_stride), -(-cols // col_stride)
    pr = max(0, (orows - 1) * row_stride + krows - rows)
    pc = max(0, (ocols - 1) * col_stride + kcols - cols)
    return orows, ocols, pr // 2, pc // 2


def conv2d_forward(x, k, row_stride=1, col_stride=1) -> np.ndarray:
    """x (C, R, W, B), k (F, C, KR, KC) -> y (F, OR, OC, B); cross-correlation, fp64 sums, one
    rounding to the input type (Conv2dNode::forward_, ginn/node/conv.h:41-49)."""
    x64, k64 = f64(x), f64(k)
    C, R, W, B = x64.shape
    F, _, KR, KC = k64.shape
    OR, OC, pt, pl = conv2d_geometry(R, W, KR, KC, row_stride, col_stride)
    xp = np.zeros((C, R + KR + row_stride, W + KC + col_stride, B))
    xp[:, pt:pt + R, pl:pl + W] = x64
    y = np.zeros((F, OR, OC, B))
    for kr in range(KR):
        for kc in range(KC):
            patch = xp[:, kr:kr + (OR - 1) * row_stride + 1:row_stride,
                       kc:kc + (OC - 1) * col_stride + 1:col_stride]
            y += np.einsum("fc,crwb->frwb", k64[:, :, kr, kc], patch)
    return y.astype(np.asarray(x).dtype)


def conv2d_backward(x, k, dy, row_stride=1, col_stride=1):
    """(dx, dk) of conv2d_forward for upstream gradient dy: the adjoints of the patch
    contraction (Conv2dNode::backward_, ginn/node/conv.h:52-64)."""
    x64, k64, dy64 = f64(x), f64(k), f64(dy)
    C, R, W, B = x64.shape
    F, _, KR, KC = k64.shape
    OR, OC, pt, pl = conv2d_geometry(R, W, KR, KC, row_stride, col_stride)
    xp = np.zeros((C, R + KR + row_stride, W + KC + col_stride, B))
    xp[:, pt:pt + R, pl:pl + W] = x64
    dxp = np.zeros_like(xp)
    dk = np.zeros_like(k64)
    for kr in range(KR):
        for kc in range(KC):
            rs = slice(kr, kr + (OR - 1) * row_stride + 1, row_stride)
            cs = slice(kc, kc + (OC - 1) * col_stride + 1, col_stride)
            dk[:, :, kr, kc] = np.einsum("frwb,crwb->fc", dy64, xp[:, rs, cs])
            dxp[:, rs, cs] += np.einsum("fc,frwb->crwb", k64[:, :, kr, kc], dy64)
    dt = np.asarray(x).dtype
    return dxp[:, pt:pt + R, pl:pl + W].astype(dt), dk.astype(dt)


def rel_frobenius(x, ref) -> float:
    x, ref = f64(x), f64(ref)
    den = np.linalg.norm(ref.ravel())
    num = np.linalg.norm((x - ref).ravel())
    return float(num / den) if den > 0 else float(num)


def elementwise_ok(x, ref, rel: float, atol: float = 1e-6) -> bool:
    """The reference's own per-element rule (test/check_node.h:104-119): within `rel`
    relatively, or both near zero."""
    x, ref = f64(x), f64(ref)
    return bool(np.all((np.abs(x - ref) <= rel * np.abs(ref)) | (np.abs(x - ref) <= atol)))


# ----------------------------------------------------------------------------------------------
# C restatement (cpu_path.c)
# ----------------------------------------------------------------------------------------------
_cpu = None


def build_cpu_path(force: bool = False) -> str:
    so = os.path.join(_HERE, "liboracle_cpu.so")
    src = os.path.join(_HERE, "cpu_path.c")
    if force or not os.path.exists(so) or os.path.getmtime(so) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "-B"], check=True, capture_output=True)
    return so


def cpu_path():
    global _cpu
    if _cpu is None:
        so = os.path.join(_HERE, "liboracle_cpu.so")
        if not os.path.exists(so):
            build_cpu_path()
        L = C.CDLL(so)
        vp, cl, ci = C.c_void_p, C.c_long, C.c_int
        L.cpu_gemm.argtypes = [ci, ci, ci, cl, cl, cl, vp, cl, vp, cl, vp, cl, ci, ci]
        L.cpu_gemm.restype = None
        L.cpu_gemm_batched.argtypes = [ci, ci, ci, cl, cl, cl, vp, cl, cl, vp, cl, cl, vp, cl, cl,
                                       cl, ci, ci]
        L.cpu_gemm_batched.restype = None
        L.cpu_max_threads.restype = ci
        _cpu = L
    return _cpu


def _dt(a: np.ndarray) -> int:
    return {np.dtype(np.float32): 0, np.dtype(np.float16): 1}[a.dtype]


def cpu_gemm(a: np.ndarray, b: np.ndarray, trans_a=False, trans_b=False,
             c: Optional[np.ndarray] = None, accumulate=False, threads: int = 1) -> np.ndarray:
    """C restatement on F-ordered arrays; returns the result in the inputs' dtype."""
    a = np.asfortranarray(a)
    b = np.asfortranarray(b)
    m = a.shape[1] if trans_a else a.shape[0]
    k = a.shape[0] if trans_a else a.shape[1]
    n = b.shape[0] if trans_b else b.shape[1]
    out = np.zeros((m, n), dtype=a.dtype, order="F") if c is None else np.asfortranarray(c).copy(order="F")
    cpu_path().cpu_gemm(_dt(a), int(trans_a), int(trans_b), m, n, k, a.ctypes.data,
                        max(a.shape[0], 1), b.ctypes.data, max(b.shape[0], 1), out.ctypes.data,
                        max(m, 1), int(accumulate), threads)
    return out
