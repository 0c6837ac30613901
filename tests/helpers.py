"""Shared helpers of the GPU parity tests: seeded inputs, tolerances, comparison."""
import numpy as np

from oracle import oracle as orc

# north-star tolerances: relative Frobenius error against the fp64 oracle
TOL = {np.dtype(np.float32): 1e-5, np.dtype(np.float16): 5e-3}
# the reference's own per-element rule (test/check_node.h:104-119, eps2 of test/nodes.cu.cpp)
ELEM = {np.dtype(np.float32): 1e-4, np.dtype(np.float16): 1e-2}


def randn(rng, shape, dtype, scale=1.0):
    return (rng.standard_normal(shape) * scale).astype(dtype)


def check(x, ref, dtype, what=""):
    e = orc.rel_frobenius(x, ref)
    assert e <= TOL[np.dtype(dtype)], f"{what}: rel Frobenius {e:.3e} > {TOL[np.dtype(dtype)]}"
    return e


def check_elementwise(x, ref, dtype, what=""):
    scale = float(np.max(np.abs(ref))) if np.size(ref) else 1.0
    assert orc.elementwise_ok(x, ref, ELEM[np.dtype(dtype)], atol=ELEM[np.dtype(dtype)] * 1e-2 * max(scale, 1e-30) + 1e-30), what
