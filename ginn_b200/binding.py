"""ctypes binding of the C ABI declared in include/ginn_b200.h.

Matrices are torch CUDA tensors viewed column-major, as ginn stores them: a (rows, cols)
tensor with strides (1, ld).  ``colmajor`` / ``from_host`` build such tensors.  Batched operands
are (rows, cols, batch) tensors with strides (1, ld, batch_stride).
"""
from __future__ import annotations

import ctypes as C
import os
from dataclasses import dataclass
from typing import Optional, Sequence

import numpy as np
import torch

F32, F16 = 0, 1
ACT_NONE, ACT_TANH, ACT_SIGMOID, ACT_RELU = 0, 1, 2, 3
GROUPED_FORWARD, GROUPED_DX, GROUPED_DW = 0, 1, 2

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libginn_b200.so")
_lib = None


class GinnB200Error(RuntimeError):
    def __init__(self, status: int, text: str):
        super().__init__(f"ginn_b200 status {status}: {text}")
        self.status = status


class _Pair(C.Structure):
    _fields_ = [("a", C.c_void_p), ("lda", C.c_int64), ("b", C.c_void_p), ("ldb", C.c_int64),
                ("k", C.c_int64)]


class _PairGrad(C.Structure):
    _fields_ = [("a", C.c_void_p), ("lda", C.c_int64), ("b", C.c_void_p), ("ldb", C.c_int64),
                ("k", C.c_int64), ("da", C.c_void_p), ("ldda", C.c_int64), ("db", C.c_void_p),
                ("lddb", C.c_int64)]


class _Group(C.Structure):
    _fields_ = [("w", C.c_void_p), ("ldw", C.c_int64), ("m", C.c_int64), ("k", C.c_int64),
                ("bias", C.c_void_p), ("ncols", C.c_int64), ("x_cols", C.POINTER(C.c_void_p)),
                ("y_cols", C.POINTER(C.c_void_p)), ("dx_cols", C.POINTER(C.c_void_p)),
                ("dw", C.c_void_p), ("lddw", C.c_int64), ("dbias", C.c_void_p),
                ("accumulate", C.c_int), ("act", C.c_int), ("out_cols", C.POINTER(C.c_void_p))]


def lib_path() -> str:
    return _LIB_PATH


def lib():
    """Loads libginn_b200.so; there is no fallback if it is missing."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(_LIB_PATH):
        raise ImportError(
            f"{_LIB_PATH} is missing: build it with `python -m ginn_b200.build` "
            "(nvcc, sm_100a). ginn_b200 has no CPU or PyTorch fallback.")
    L = C.CDLL(_LIB_PATH)
    i64, vp, ci = C.c_int64, C.c_void_p, C.c_int
    L.ginn_b200_gemm.argtypes = [ci, vp, ci, ci, ci, i64, i64, i64, vp, i64, vp, i64, vp, i64, ci]
    L.ginn_b200_gemm_batched.argtypes = [ci, vp, ci, ci, ci, i64, i64, i64, vp, i64, i64, vp, i64,
                                         i64, vp, i64, i64, i64, ci]
    L.ginn_b200_prod_backward.argtypes = [ci, vp, ci, i64, i64, i64, i64, vp, i64, i64, vp, i64, i64,
                                          vp, i64, i64, vp, i64, i64, vp, i64, i64]
    L.ginn_b200_prod_backward.restype = ci
    L.ginn_b200_affine_forward.argtypes = [ci, vp, ci, ci, C.POINTER(_Pair), i64, i64, vp, ci, vp,
                                           i64]
    L.ginn_b200_affine_backward.argtypes = [ci, vp, ci, ci, C.POINTER(_PairGrad), i64, i64, vp,
                                            i64, vp, i64, ci, vp]
    L.ginn_b200_affine_backward_scratch.argtypes = [ci, vp, ci, ci, C.POINTER(_PairGrad), i64, i64,
                                                    vp, i64, vp, i64, ci, vp, vp]
    L.ginn_b200_affine_backward_scratch.restype = ci
    L.ginn_b200_grouped.argtypes = [ci, vp, ci, ci, ci, C.POINTER(_Group)]
    L.ginn_b200_grouped_static.argtypes = [ci, vp, ci, ci, ci, C.POINTER(_Group)]
    L.ginn_b200_grouped_static.restype = ci
    L.ginn_b200_grouped_static_status.argtypes = [ci, ci]
    L.ginn_b200_grouped_static_status.restype = ci
    L.ginn_b200_level_create.argtypes = [ci, ci, ci, ci, C.POINTER(_Group), C.POINTER(vp)]
    L.ginn_b200_level_run.argtypes = [vp, vp]
    L.ginn_b200_level_destroy.argtypes = [vp]
    for name in ("ginn_b200_level_create", "ginn_b200_level_run", "ginn_b200_level_destroy"):
        getattr(L, name).restype = ci
    cf, fp = C.c_float, C.POINTER(C.c_float)
    L.ginn_b200_pick_nll_forward.argtypes = [ci, vp, ci, i64, i64, vp, i64, vp, vp, i64, vp]
    L.ginn_b200_pick_nll_backward.argtypes = [ci, vp, ci, i64, i64, vp, i64, vp, vp, vp, i64]
    L.ginn_b200_adam_update.argtypes = [ci, vp, ci, i64, vp, vp, vp, vp, cf, cf, cf, cf, cf, cf, cf]
    L.ginn_b200_softmax_forward.argtypes = [ci, vp, ci, i64, i64, vp, i64, vp, i64]
    L.ginn_b200_softmax_backward.argtypes = [ci, vp, ci, i64, i64, vp, i64, vp, i64, vp, i64, ci]
    L.ginn_b200_lstm_cell_forward.argtypes = [ci, vp, i64, i64, i64, vp, i64, vp, i64, vp, i64, vp,
                                              i64, vp, i64]
    L.ginn_b200_lstm_cell_backward.argtypes = [ci, vp, i64, i64, i64, vp, i64, vp, i64, vp, i64, vp,
                                               i64, vp, i64, cf, vp, i64, vp, i64]
    L.ginn_b200_lstm_cell_forward.restype = L.ginn_b200_lstm_cell_backward.restype = ci
    L.ginn_b200_lstm_cells.argtypes = [ci, vp, ci, i64, i64, C.POINTER(vp)]
    L.ginn_b200_lstm_cells.restype = ci
    for name in ("ginn_b200_pick_nll_forward", "ginn_b200_pick_nll_backward",
                 "ginn_b200_adam_update", "ginn_b200_softmax_forward",
                 "ginn_b200_softmax_backward"):
        getattr(L, name).restype = ci
    L.ginn_b200_attention_forward.argtypes = [ci, vp, ci, i64, i64, i64, vp, i64, i64, vp, i64, i64,
                                              vp, i64, i64, cf, ci, vp, i64, i64, vp, i64, i64]
    L.ginn_b200_attention_backward.argtypes = [ci, vp, ci, i64, i64, i64, vp, i64, i64, vp, i64, i64,
                                               vp, i64, i64, cf, vp, i64, i64, vp, i64, i64, vp, vp,
                                               vp, vp]
    L.ginn_b200_attention_forward.restype = L.ginn_b200_attention_backward.restype = ci
    L.ginn_b200_conv2d_workspace.argtypes = [ci] + [i64] * 9
    L.ginn_b200_conv2d_workspace.restype = C.c_size_t
    L.ginn_b200_conv2d_forward.argtypes = [ci, vp, ci] + [i64] * 9 + [vp, vp, vp, vp]
    L.ginn_b200_conv2d_backward.argtypes = [ci, vp, ci] + [i64] * 9 + [vp, vp, vp, vp, vp, vp]
    L.ginn_b200_conv2d_forward.restype = L.ginn_b200_conv2d_backward.restype = ci
    L.ginn_b200_fill.argtypes = [ci, vp, ci, i64, vp, cf]
    L.ginn_b200_fill.restype = ci
    L.ginn_b200_last_error.restype = C.c_char_p
    L.ginn_b200_device_status.argtypes = [ci, ci]
    L.ginn_b200_set_option.argtypes = [C.c_char_p, ci]
    L.ginn_b200_launch_count.restype = i64
    for name in ("ginn_b200_gemm", "ginn_b200_gemm_batched", "ginn_b200_affine_forward",
                 "ginn_b200_affine_backward", "ginn_b200_grouped", "ginn_b200_device_status",
                 "ginn_b200_version", "ginn_b200_set_option"):
        getattr(L, name).restype = ci
    _lib = L
    return L


def _check(status: int):
    if status != 0:
        raise GinnB200Error(status, lib().ginn_b200_last_error().decode())


def _dtype_of(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return F32
    if t.dtype == torch.float16:
        return F16
    raise GinnB200Error(2, f"unsupported tensor dtype {t.dtype}")


def _stream(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def _dev(t: torch.Tensor) -> int:
    return t.device.index if t.device.index is not None else torch.cuda.current_device()


def _ld(t: torch.Tensor) -> int:
    assert t.dim() >= 2 and (t.shape[0] <= 1 or t.stride(0) == 1), "matrix must be column-major"
    return max(int(t.stride(1)) if t.shape[1] > 1 else int(t.shape[0]), 1)


def colmajor(rows: int, cols: int, dtype, device="cuda", ld: Optional[int] = None,
             batches: Optional[int] = None, fill: Optional[float] = None) -> torch.Tensor:
    """Uninitialised (or filled) column-major matrix, optionally padded (ld) or batched."""
    ld = rows if ld is None else ld
    n = ld * cols * (batches or 1)
    buf = torch.empty(max(n, 1), dtype=dtype, device=device)
    if fill is not None:
        buf.fill_(fill)
    if batches is None:
        return torch.as_strided(buf, (rows, cols), (1, ld))
    return torch.as_strided(buf, (rows, cols, batches), (1, ld, ld * cols))


def from_host(a: np.ndarray, device="cuda", ld: Optional[int] = None) -> torch.Tensor:
    """numpy (rows, cols[, batch]) array -> column-major torch tensor on the GPU."""
    tdt = {np.dtype(np.float32): torch.float32, np.dtype(np.float16): torch.float16}[a.dtype]
    if a.ndim == 1:
        return torch.from_numpy(np.ascontiguousarray(a)).to(device)
    if a.ndim == 2:
        out = colmajor(a.shape[0], a.shape[1], tdt, device, ld)
    else:
        out = colmajor(a.shape[0], a.shape[1], tdt, device, ld, a.shape[2])
    out.copy_(torch.from_numpy(np.ascontiguousarray(a)))
    return out


def to_host(t: torch.Tensor) -> np.ndarray:
    return t.detach().cpu().numpy()


def gemm(a: torch.Tensor, b: torch.Tensor, c: torch.Tensor, trans_a=False, trans_b=False,
         accumulate=False) -> torch.Tensor:
    """c = op(a) @ op(b) (+ c).  Mirrors internal::gpu_prod (ginn/prod.h:211-253)."""
    m, n = c.shape
    k = a.shape[0] if trans_a else a.shape[1]
    _check(lib().ginn_b200_gemm(_dev(c), _stream(c), _dtype_of(c), int(trans_a), int(trans_b), m,
                                n, k, a.data_ptr(), _ld(a), b.data_ptr(), _ld(b), c.data_ptr(),
                                _ld(c), int(accumulate)))
    return c


def gemm_batched(a, b, c, trans_a=False, trans_b=False, accumulate=False):
    """c[:,:,i] = op(a[:,:,i]) @ op(b[:,:,i]) (+ c[:,:,i]); internal::gpu_batched_prod
    (ginn/prod.h:255-310)."""
    m, n, batches = c.shape
    k = a.shape[0] if trans_a else a.shape[1]
    sa = a.stride(2) if batches > 1 else a.shape[0] * a.shape[1]
    sb = b.stride(2) if batches > 1 else b.shape[0] * b.shape[1]
    sc = c.stride(2) if batches > 1 else c.shape[0] * c.shape[1]
    _check(lib().ginn_b200_gemm_batched(
        _dev(c), _stream(c), _dtype_of(c), int(trans_a), int(trans_b), m, n, k, a.data_ptr(),
        _ld(a), sa, b.data_ptr(), _ld(b), sb, c.data_ptr(), _ld(c), sc, batches, int(accumulate)))
    return c


def prod_backward(a, b, dc, da=None, db=None) -> None:
    """Both gradient products of c = a @ b (per batch for rank-3 tensors): da += dc @ b^T,
    db += a^T @ dc; ProdNode::backward_ / BatchedProdNode::backward_ (ginn/node/prod.h:51-66,
    118-130)."""
    batched = a.dim() == 3
    m, k = a.shape[0], a.shape[1]
    n = b.shape[1]
    batches = a.shape[2] if batched else 1
    st = lambda t: 0 if t is None else (t.stride(2) if batched and batches > 1 else t.shape[0] * t.shape[1])
    ld = lambda t: 0 if t is None else _ld(t)
    _check(lib().ginn_b200_prod_backward(
        _dev(dc), _stream(dc), _dtype_of(dc), m, n, k, batches, a.data_ptr(), _ld(a), st(a),
        b.data_ptr(), _ld(b), st(b), dc.data_ptr(), _ld(dc), st(dc), _ptr(da), ld(da), st(da),
        _ptr(db), ld(db), st(db)))


@dataclass
class Pair:
    a: torch.Tensor
    b: torch.Tensor


@dataclass
class PairGrad:
    a: torch.Tensor
    b: torch.Tensor
    da: Optional[torch.Tensor] = None
    db: Optional[torch.Tensor] = None


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def affine_forward(pairs: Sequence[Pair], bias: Optional[torch.Tensor], act: int,
                   out: torch.Tensor) -> torch.Tensor:
    """out = act(sum_i a_i @ b_i + bias); AffineNode::forward_ (ginn/node/affine.h:35-77)."""
    arr = (_Pair * len(pairs))()
    for i, p in enumerate(pairs):
        arr[i] = _Pair(p.a.data_ptr(), _ld(p.a), p.b.data_ptr(), _ld(p.b), p.a.shape[1])
    m, n = out.shape
    _check(lib().ginn_b200_affine_forward(_dev(out), _stream(out), _dtype_of(out), len(pairs), arr,
                                          m, n, _ptr(bias), act, out.data_ptr(), _ld(out)))
    return out


def affine_backward(pairs: Sequence[PairGrad], dout: torch.Tensor, out: Optional[torch.Tensor],
                    act: int, dbias: Optional[torch.Tensor],
                    scratch: Optional[torch.Tensor] = None) -> None:
    """AffineNode::backward_ (ginn/node/affine.h:79-129): accumulates into da/db/dbias.  `scratch`
    (m x n, the node's d-pre-activation tensor) makes the Half path allocation-free."""
    arr = (_PairGrad * max(len(pairs), 1))()
    for i, p in enumerate(pairs):
        arr[i] = _PairGrad(p.a.data_ptr(), _ld(p.a), p.b.data_ptr(), _ld(p.b), p.a.shape[1],
                           _ptr(p.da), _ld(p.da) if p.da is not None else 0, _ptr(p.db),
                           _ld(p.db) if p.db is not None else 0)
    m, n = dout.shape
    _check(lib().ginn_b200_affine_backward_scratch(
        _dev(dout), _stream(dout), _dtype_of(dout), len(pairs), arr, m, n, dout.data_ptr(),
        _ld(dout), _ptr(out), _ld(out) if out is not None else 0, act, _ptr(dbias), _ptr(scratch)))


@dataclass
class Group:
    """One autobatch group: shared W (m x k) and per-node column vectors."""
    w: torch.Tensor
    x_cols: Sequence[torch.Tensor] = ()   # each (k,)
    y_cols: Sequence[torch.Tensor] = ()   # each (m,): outputs (forward) or upstream grads
    dx_cols: Sequence[torch.Tensor] = ()  # each (k,)
    bias: Optional[torch.Tensor] = None
    dw: Optional[torch.Tensor] = None
    dbias: Optional[torch.Tensor] = None
    accumulate: bool = False              # forward: y += W x (+ bias)
    act: int = ACT_NONE                   # forward: fused nonlinearity; dX / dW: its derivative
    out_cols: Sequence[torch.Tensor] = () # dX / dW with act: the nodes' forward values (m,)


def grouped_static(mode: int, groups: Sequence[Group]) -> None:
    """`grouped` through the entry point that allocates nothing (fixed 256 KiB descriptor array
    inside the library); for hosts that may not call the CUDA allocator."""
    _grouped_call(lib().ginn_b200_grouped_static, mode, groups)


def grouped(mode: int, groups: Sequence[Group]) -> None:
    """All groups of one autobatch level in one launch (ginn/autobatch.h:149-183)."""
    _grouped_call(lib().ginn_b200_grouped, mode, groups)


def _build_groups(groups: Sequence[Group]):
    """ctypes image of a level: the group array plus the pointer tables it refers to."""
    arr = (_Group * len(groups))()
    keep = []

    def table(ts):
        t = (C.c_void_p * max(len(ts), 1))(*[x.data_ptr() for x in ts])
        keep.append(t)
        return C.cast(t, C.POINTER(C.c_void_p))

    for i, g in enumerate(groups):
        m, k = g.w.shape
        ncols = len(g.y_cols)
        arr[i] = _Group(g.w.data_ptr(), _ld(g.w), m, k, _ptr(g.bias), ncols,
                        table(g.x_cols) if len(g.x_cols) else None, table(g.y_cols),
                        table(g.dx_cols) if len(g.dx_cols) else None, _ptr(g.dw),
                        _ld(g.dw) if g.dw is not None else 0, _ptr(g.dbias),
                        int(g.accumulate), int(g.act),
                        table(g.out_cols) if len(g.out_cols) else None)
    return arr, keep


def _grouped_call(fn, mode: int, groups: Sequence[Group]) -> None:
    if not groups:
        return
    arr, _keep = _build_groups(groups)
    w0 = groups[0].w
    _check(fn(_dev(w0), _stream(w0), _dtype_of(w0), mode, len(groups), arr))


class GroupedCall:
    """A level prepared once and launched many times (ginn_b200_level_*): descriptors and column
    tables stay resident on the device, a call is one kernel launch.  The tensors must stay
    alive and in place, as the nodes of a re-evaluated ginn graph do.  With static=True the
    allocation-free entry point is used instead (tables rebuilt from the kept host arrays)."""

    def __init__(self, mode: int, groups: Sequence[Group], static: bool = False):
        self.mode, self.n = mode, len(groups)
        self.groups = list(groups)
        self.arr, self._keep = _build_groups(groups)
        w0 = groups[0].w
        self.dev, self.dtype, self.w0 = _dev(w0), _dtype_of(w0), w0
        self.static = static
        self.handle = None
        if not static:
            h = C.c_void_p()
            _check(lib().ginn_b200_level_create(self.dev, self.dtype, mode, self.n, self.arr,
                                                C.byref(h)))
            self.handle = h

    def __call__(self):
        if self.static:
            _check(lib().ginn_b200_grouped_static(self.dev, _stream(self.w0), self.dtype,
                                                  self.mode, self.n, self.arr))
        else:
            _check(lib().ginn_b200_level_run(self.handle, _stream(self.w0)))

    def run(self, stream: int):
        """Same as calling the object, on an explicit stream handle (saves the per-call lookup
        of torch's current stream in launch-bound loops)."""
        if self.static:
            _check(lib().ginn_b200_grouped_static(self.dev, stream, self.dtype, self.mode, self.n,
                                                  self.arr))
        else:
            _check(_lib.ginn_b200_level_run(self.handle, stream))

    def __del__(self):
        if getattr(self, "handle", None) is not None and _lib is not None:
            _lib.ginn_b200_level_destroy(self.handle)
            self.handle = None


def pick_nll_forward(x: torch.Tensor, index: torch.Tensor, smax: torch.Tensor,
                     value: torch.Tensor) -> None:
    """smax = column softmax of x; value[j] = -log smax[index[j], j]  (ginn_b200_pick_nll_forward).
    x, smax: column-major rows x cols; index: int32 (cols); value: cols elements."""
    assert index.dtype == torch.int32 and index.is_contiguous() and value.is_contiguous()
    rows, cols = x.shape
    _check(lib().ginn_b200_pick_nll_forward(_dev(x), _stream(x), _dtype_of(x), rows, cols,
                                            x.data_ptr(), _ld(x), index.data_ptr(),
                                            smax.data_ptr(), _ld(smax), value.data_ptr()))


def pick_nll_backward(smax: torch.Tensor, index: torch.Tensor, grad: torch.Tensor,
                      dx: torch.Tensor) -> None:
    """dx += (smax - onehot(index)) * grad  (ginn_b200_pick_nll_backward)."""
    assert index.dtype == torch.int32 and index.is_contiguous() and grad.is_contiguous()
    rows, cols = smax.shape
    _check(lib().ginn_b200_pick_nll_backward(_dev(smax), _stream(smax), _dtype_of(smax), rows, cols,
                                             smax.data_ptr(), _ld(smax), index.data_ptr(),
                                             grad.data_ptr(), dx.data_ptr(), _ld(dx)))


def _fold_cols(t: torch.Tensor):
    """(rows, cols) of a column-major tensor with its trailing dimensions folded into cols."""
    assert t.stride(0) == 1 and (t.dim() < 3 or t.stride(2) == t.stride(1) * t.shape[1])
    return t.shape[0], t.numel() // t.shape[0]


def softmax_forward(x: torch.Tensor, y: torch.Tensor) -> None:
    """y = softmax over dimension 0 of x (column-major, batches folded into the columns)."""
    rows, cols = _fold_cols(x)
    _check(lib().ginn_b200_softmax_forward(_dev(x), _stream(x), _dtype_of(x), rows, cols,
                                           x.data_ptr(), _ld(x), y.data_ptr(), _ld(y)))


def softmax_backward(y: torch.Tensor, dy: torch.Tensor, dx: torch.Tensor, accumulate=True) -> None:
    """dx (+)= y * (dy - sum over dimension 0 of y * dy)."""
    rows, cols = _fold_cols(y)
    _check(lib().ginn_b200_softmax_backward(_dev(y), _stream(y), _dtype_of(y), rows, cols,
                                            y.data_ptr(), _ld(y), dy.data_ptr(), _ld(dy),
                                            dx.data_ptr(), _ld(dx), int(accumulate)))


def lstm_cell_forward(gates, c_prev, c, h, xh_next=None, n_next=0) -> None:
    """Cell update of one level (ginn_b200_lstm_cell_forward): gates (4H x n) are replaced by
    their activations; c_prev may be None; xh_next: the next level's h block (H x n_next view)."""
    H, n = c.shape
    _check(lib().ginn_b200_lstm_cell_forward(
        _dev(c), _stream(c), H, n, n_next if xh_next is not None else 0, gates.data_ptr(),
        _ld(gates), _ptr(c_prev), _ld(c_prev) if c_prev is not None else 0, c.data_ptr(), _ld(c),
        h.data_ptr(), _ld(h), _ptr(xh_next), _ld(xh_next) if xh_next is not None else 0))


def lstm_cell_backward(gates, c, c_prev, dh_next, dc_next, n_next, dgates, dc_out, dh_end=1.0) -> None:
    """Gradients of one level's cell update (ginn_b200_lstm_cell_backward)."""
    H, n = c.shape
    _check(lib().ginn_b200_lstm_cell_backward(
        _dev(c), _stream(c), H, n, n_next, gates.data_ptr(), _ld(gates), c.data_ptr(), _ld(c),
        _ptr(c_prev), _ld(c_prev) if c_prev is not None else 0, _ptr(dh_next),
        _ld(dh_next) if dh_next is not None else 0, _ptr(dc_next),
        _ld(dc_next) if dc_next is not None else 0, dh_end, dgates.data_ptr(), _ld(dgates),
        dc_out.data_ptr(), _ld(dc_out)))


def lstm_cells(backward: bool, tables: Sequence[Sequence[Optional[torch.Tensor]]]) -> None:
    """Cell update over per-cell tensors (ginn_b200_lstm_cells): `tables` = 4 (forward: gates,
    c_prev, c, h) or 7 (backward: gates, c, c_prev, dh, dc, dgates, dc_prev) lists with one
    tensor (or None where allowed) per cell.  hidden = len(c) of the first cell."""
    n = len(tables[0])
    flat = (C.c_void_p * (len(tables) * n))(*[_ptr(t) for tab in tables for t in tab])
    some = tables[0][0]
    hidden = some.numel() // 4
    _check(lib().ginn_b200_lstm_cells(_dev(some), _stream(some), int(backward), hidden, n, flat))


def _bstride(t: torch.Tensor) -> int:
    return int(t.stride(2)) if t.shape[2] > 1 else int(t.shape[1]) * _ld(t)


def attention_forward(k, q, v, o, p=None, scale=1.0, causal=False) -> None:
    """o = v @ softmax(scale * k @ q [masked]) per batch (ginn_b200_attention_forward).  k: (T, hs,
    nb); q, v, o: (hs, T, nb); p: (T, T, nb) or None; column-major batched tensors."""
    T, hs, nb = k.shape
    _check(lib().ginn_b200_attention_forward(
        _dev(k), _stream(k), _dtype_of(k), T, hs, nb, k.data_ptr(), _ld(k), _bstride(k), q.data_ptr(),
        _ld(q), _bstride(q), v.data_ptr(), _ld(v), _bstride(v), scale, int(causal), o.data_ptr(),
        _ld(o), _bstride(o), _ptr(p), _ld(p) if p is not None else 0,
        _bstride(p) if p is not None else 0))


def attention_backward(k, q, v, p, d_o, ds, dk=None, dq=None, dv=None, scale=1.0) -> None:
    """dk += ..., dq += ..., dv += ... from the kept softmax output p (ginn_b200_attention_backward);
    ds: scratch shaped like p."""
    T, hs, nb = k.shape
    _check(lib().ginn_b200_attention_backward(
        _dev(k), _stream(k), _dtype_of(k), T, hs, nb, k.data_ptr(), _ld(k), _bstride(k), q.data_ptr(),
        _ld(q), _bstride(q), v.data_ptr(), _ld(v), _bstride(v), scale, p.data_ptr(), _ld(p), _bstride(p),
        d_o.data_ptr(), _ld(d_o), _bstride(d_o), ds.data_ptr(), _ptr(dk), _ptr(dq), _ptr(dv)))


def _conv_dims(x: torch.Tensor, k: torch.Tensor):
    """Extents of contiguous column-major tensors given as torch tensors whose dimensions are
    listed in ginn's order (channels, rows, cols, batch) / (filters, channels, krows, kcols) and
    whose strides put the first dimension fastest."""
    for t in (x, k):
        want, acc = [], 1
        for d in t.shape:
            want.append(acc)
            acc *= d
        assert list(t.stride()) == want, "convolution tensors must be column-major and contiguous"
    return tuple(x.shape) + (k.shape[0], k.shape[2], k.shape[3])


def colmajor_nd(shape, dtype, device="cuda", fill: Optional[float] = None) -> torch.Tensor:
    """Contiguous column-major tensor of any rank (first dimension fastest)."""
    n = 1
    strides = []
    for d in shape:
        strides.append(n)
        n *= d
    buf = torch.empty(max(n, 1), dtype=dtype, device=device)
    if fill is not None:
        buf.fill_(fill)
    return torch.as_strided(buf, tuple(shape), tuple(strides))


def from_host_nd(a: np.ndarray, device="cuda") -> torch.Tensor:
    tdt = {np.dtype(np.float32): torch.float32, np.dtype(np.float16): torch.float16}[a.dtype]
    out = colmajor_nd(a.shape, tdt, device)
    out.copy_(torch.from_numpy(np.ascontiguousarray(a)))
    return out


def conv2d_workspace_bytes(x, k, row_stride=1, col_stride=1) -> int:
    dims = _conv_dims(x, k)
    return int(lib().ginn_b200_conv2d_workspace(_dtype_of(x), *dims, row_stride, col_stride))


def conv2d_forward(x, k, y, row_stride=1, col_stride=1, workspace: Optional[torch.Tensor] = None):
    """y = Conv2d(x, k) with SAME padding (ginn_b200_conv2d_forward); Conv2dNode::forward_."""
    dims = _conv_dims(x, k)
    _check(lib().ginn_b200_conv2d_forward(_dev(x), _stream(x), _dtype_of(x), *dims, row_stride,
                                          col_stride, x.data_ptr(), k.data_ptr(), y.data_ptr(),
                                          _ptr(workspace)))
    return y


def conv2d_backward(x, k, dy, dx=None, dk=None, row_stride=1, col_stride=1,
                    workspace: Optional[torch.Tensor] = None) -> None:
    """dx += ..., dk += ... (ginn_b200_conv2d_backward); Conv2dNode::backward_."""
    dims = _conv_dims(x, k)
    _check(lib().ginn_b200_conv2d_backward(_dev(x), _stream(x), _dtype_of(x), *dims, row_stride,
                                           col_stride, x.data_ptr(), k.data_ptr(), dy.data_ptr(),
                                           _ptr(dx), _ptr(dk), _ptr(workspace)))


def fill(x: torch.Tensor, value: float) -> None:
    """x[...] = value for a contiguous tensor (ginn_b200_fill)."""
    assert x.is_contiguous() or x.T.is_contiguous()
    _check(lib().ginn_b200_fill(_dev(x), _stream(x), _dtype_of(x), x.numel(), x.data_ptr(), value))


def adam_update(w: torch.Tensor, d: torch.Tensor, m: torch.Tensor, v: torch.Tensor, t: int,
                lr=1e-3, clip=5.0, eps=1e-8, beta1=0.9, beta2=0.999) -> None:
    """Step t (1-based) of Adam on flat contiguous tensors (ginn_b200_adam_update); m, v fp32."""
    assert w.is_contiguous() and d.is_contiguous() and m.dtype == torch.float32 == v.dtype
    assert w.numel() == d.numel() == m.numel() == v.numel()
    _check(lib().ginn_b200_adam_update(_dev(w), _stream(w), _dtype_of(w), w.numel(), w.data_ptr(),
                                       d.data_ptr(), m.data_ptr(), v.data_ptr(), lr, clip, eps,
                                       beta1, beta2, beta1 ** t, beta2 ** t))


def device_status(device: int = 0, reset: bool = True) -> int:
    return lib().ginn_b200_device_status(device, int(reset))


def grouped_static_status(device: int = 0, reset: bool = True) -> int:
    """Status word of the kernels launched through `grouped_static` (0 = healthy)."""
    return lib().ginn_b200_grouped_static_status(device, int(reset))


def set_option(name: str, value: int) -> None:
    _check(lib().ginn_b200_set_option(name.encode(), value))


def launch_count() -> int:
    return int(lib().ginn_b200_launch_count())


def selftest(device: int = 0) -> None:
    """Bounded-wait self test (ginn_b200_selftest); raises if the time-out is not reported."""
    fn = lib().ginn_b200_selftest
    fn.argtypes, fn.restype = [C.c_int], C.c_int
    _check(fn(device))


def version() -> int:
    return lib().ginn_b200_version()
