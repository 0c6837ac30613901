"""ginn_b200: B200 (sm_100a) back end for ginn's Affine / Prod / BatchedProd / autobatch GEMMs.

The product is the shared library ``libginn_b200.so`` (C ABI in ``include/ginn_b200.h``) and
the header-only C++ layer in ``ginn_b200/include``.  This Python package is a thin ctypes
binding used by the tests and the benchmark; it never computes anything itself and raises if
the CUDA library is missing.
"""
from .binding import (  # noqa: F401
    ACT_NONE, ACT_RELU, ACT_SIGMOID, ACT_TANH, F16, F32, GinnB200Error, Group, GroupedCall, Pair,
    PairGrad,
    adam_update, affine_backward, attention_backward, attention_forward, colmajor_nd, conv2d_backward, conv2d_forward, conv2d_workspace_bytes, from_host_nd, affine_forward, device_status, fill, gemm, gemm_batched, grouped, grouped_static, grouped_static_status, launch_count,
    lib, lib_path, lstm_cell_backward, lstm_cell_forward, lstm_cells, pick_nll_backward, pick_nll_forward, prod_backward, selftest, set_option, softmax_backward, softmax_forward, version,
)
