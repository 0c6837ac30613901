"""GPU parity of ginn_b200_gemm / ginn_b200_gemm_batched (through the C ABI) against the oracle.

Mirrors the reference's CPU-vs-GPU protocol (test/check_node.h:27-121): identical inputs, every
output within tolerance, accumulation (`+=`) checked by running a product twice into one buffer.
"""
import numpy as np
import pytest
import torch

from oracle import oracle as orc
from ginn_b200 import binding as B
from helpers import check, check_elementwise, randn

pytestmark = pytest.mark.gpu

SHAPES = [(1, 1, 1), (2, 2, 3), (5, 7, 9), (16, 16, 16), (17, 33, 65), (31, 63, 127),
          (64, 64, 64), (65, 129, 33), (128, 128, 32), (128, 32, 128), (130, 70, 300),
          (129, 257, 100), (512, 128, 784)]
TRANS = [(False, False), (True, False), (False, True), (True, True)]


def run_gemm(gb, rng, dt, m, n, k, ta, tb, acc, ld_pad=0, offset=0):
    a = randn(rng, (k, m) if ta else (m, k), dt)
    b = randn(rng, (n, k) if tb else (k, n), dt)
    c0 = randn(rng, (m, n), dt)
    if ld_pad or offset:
        def place(x):
            t = B.colmajor(x.shape[0], x.shape[1] + 1, torch.from_numpy(x[:1, :1]).dtype,
                           ld=x.shape[0] + ld_pad)
            v = torch.as_strided(t, x.shape, (1, x.shape[0] + ld_pad), storage_offset=offset)
            v.copy_(torch.from_numpy(x))
            return v
        A, Bm, C = place(a), place(b), place(c0)
    else:
        A, Bm, C = B.from_host(a), B.from_host(b), B.from_host(c0)
    gb.gemm(A, Bm, C, ta, tb, acc)
    torch.cuda.synchronize()
    ref = orc.gemm(a, b, ta, tb, c0, acc)
    got = B.to_host(C)
    check(got, ref, dt, f"m{m} n{n} k{k} ta{ta} tb{tb} acc{acc}")
    return got, ref


@pytest.mark.parametrize("dt", [np.float32, np.float16])
@pytest.mark.parametrize("path", [0, 5])
def test_shape_sweep_all_transposes(gpu, dt, path):
    gpu.set_option("force_path", path)
    rng = np.random.default_rng(11)
    for (m, n, k) in SHAPES:
        for ta, tb in TRANS:
            run_gemm(gpu, rng, dt, m, n, k, ta, tb, False)
    for ta, tb in TRANS:
        run_gemm(gpu, rng, dt, 130, 70, 300, ta, tb, True)


@pytest.mark.parametrize("dt", [np.float32, np.float16])
@pytest.mark.parametrize("path", [0, 5])
def test_padded_leading_dimension_and_unaligned_base(gpu, dt, path):
    """ginn's PreallocGpu hands out unaligned bump pointers (ginn/dev.h:237-245) and
    RowwiseUncat views start at arbitrary column offsets (ginn/node/layout.h:283-289)."""
    gpu.set_option("force_path", path)
    rng = np.random.default_rng(12)
    for (m, n, k) in [(37, 41, 53), (128, 64, 96), (200, 100, 260)]:
        for ta, tb in TRANS[:3]:
            for pad, off in [(3, 0), (0, 1), (5, 3)]:
                run_gemm(gpu, rng, dt, m, n, k, ta, tb, True, pad, off)


@pytest.mark.parametrize("dt", [np.float32, np.float16])
def test_reference_elementwise_rule(gpu, dt):
    """WithinRel(cpu, eps2) per element, as check_expr does, on a well-scaled product."""
    rng = np.random.default_rng(13)
    a = np.abs(randn(rng, (96, 200), dt)) + 0.5
    b = np.abs(randn(rng, (200, 80), dt)) + 0.5
    C = B.colmajor(96, 80, B.from_host(a).dtype, fill=0.0)
    gpu.gemm(B.from_host(a), B.from_host(b), C)
    torch.cuda.synchronize()
    check_elementwise(B.to_host(C), orc.gemm(a, b), dt)


def test_prod_known_answer(gpu, kat):
    """test/nodes.cu.cpp:1023-1041 through every path that accepts the shape."""
    p = kat["prod"]
    for dt, eps in [(np.float32, kat["eps"]["f32"]), (np.float16, kat["eps"]["f16_prod"])]:
        for path in (0, 3, 5):
            gpu.set_option("force_path", path)
            W, V = np.asarray(p["W"], dt), np.asarray(p["V"], dt)
            C = B.colmajor(2, 2, B.from_host(W).dtype, fill=0.0)
            gpu.gemm(B.from_host(W), B.from_host(V), C)
            torch.cuda.synchronize()
            np.testing.assert_allclose(B.to_host(C), np.asarray(p["WV"]), rtol=max(eps, 2e-6), atol=1e-6)


@pytest.mark.parametrize("dt", [np.float32, np.float16])
def test_batched_against_per_slice_products(gpu, dt):
    """test/nodes.cu.cpp:1043-1115, plus the attention shapes of min-GPT scaled down."""
    rng = np.random.default_rng(14)
    cases = [((2, 3, 4), (3, 5, 4), False, False), ((64, 16, 6), (16, 64, 6), False, False),
             ((64, 16, 6), (64, 48, 6), True, False), ((64, 16, 5), (48, 16, 5), False, True),
             ((256, 64, 8), (64, 256, 8), False, False), ((64, 256, 8), (256, 256, 8), False, False)]
    for sa, sb, ta, tb in cases:
        a, b = randn(rng, sa, dt) + 1, randn(rng, sb, dt) - 1
        m = sa[1] if ta else sa[0]
        n = sb[0] if tb else sb[1]
        c0 = randn(rng, (m, n, sa[2]), dt)
        for acc in (False, True):
            C = B.from_host(c0)
            gpu.gemm_batched(B.from_host(a), B.from_host(b), C, ta, tb, acc)
            torch.cuda.synchronize()
            check(B.to_host(C), orc.gemm_batched(a, b, ta, tb, c0, acc), dt, f"{sa}x{sb}")


def test_batched_high_rank_folds_to_three(gpu):
    rng = np.random.default_rng(15)
    a, b = randn(rng, (2, 3, 2, 2), np.float32), randn(rng, (3, 5, 2, 2), np.float32)
    a3 = a.reshape(orc.fold3(a.shape), order="F")
    b3 = b.reshape(orc.fold3(b.shape), order="F")
    C = B.colmajor(2, 5, torch.float32, batches=4, fill=0.0)
    gpu.gemm_batched(B.from_host(a3), B.from_host(b3), C)
    torch.cuda.synchronize()
    got = B.to_host(C).reshape((2, 5, 2, 2), order="F")
    for i in range(2):
        for j in range(2):
            np.testing.assert_allclose(got[:, :, i, j], a[:, :, i, j] @ b[:, :, i, j], rtol=1e-5, atol=1e-6)


def test_batched_dot_products_of_softmax_backward(gpu):
    """m = n = 1 batched products (ginn/nonlin.h:180-183, ginn/node/layernorm.h:61-64)."""
    rng = np.random.default_rng(16)
    rows, cols = 50, 3000
    y, dy = randn(rng, (rows, cols), np.float32), randn(rng, (rows, cols), np.float32)
    out = B.colmajor(1, 1, torch.float32, batches=cols, fill=0.0)
    gpu.gemm_batched(B.from_host(y.reshape(1, rows, cols)), B.from_host(dy.reshape(rows, 1, cols)), out)
    torch.cuda.synchronize()
    check(B.to_host(out).ravel(), (y.astype(np.float64) * dy).sum(0), np.float32)


@pytest.mark.parametrize("trans", TRANS[:3])
@pytest.mark.parametrize("path", [2, 4])
def test_tma_path_half(gpu, trans, path):
    """Path 2: one CTA per 128 x 256 tile; path 4: CTA pairs (cta_group::2) on 256 x 256 tiles."""
    gpu.set_option("force_path", path)
    rng = np.random.default_rng(17)
    ta, tb = trans
    for (m, n, k) in [(128, 256, 64), (136, 264, 72), (256, 512, 512), (384, 256, 1000)]:
        for acc in (False, True):
            run_gemm(gpu, rng, np.float16, m, n, k, ta, tb, acc)
    a, b = randn(rng, (256, 128, 5), np.float16), randn(rng, (128, 256, 5), np.float16)
    C = B.colmajor(256, 256, torch.float16, batches=5, fill=0.0)
    gpu.gemm_batched(B.from_host(a), B.from_host(b), C)
    torch.cuda.synchronize()
    check(B.to_host(C), orc.gemm_batched(a, b), np.float16)


def test_pair_kernel_l2_hints_do_not_change_results(gpu):
    """The CTA-pair kernel's L2 eviction hints only steer caching: the same product with and
    without them must agree bit for bit, with and without accumulation."""
    gpu.set_option("force_path", 4)
    rng = np.random.default_rng(23)
    a, b = randn(rng, (512, 320), np.float16), randn(rng, (768, 320), np.float16)
    c0 = randn(rng, (512, 768), np.float16)
    outs = []
    try:
        for hint in (0, 1, 2, 3):
            gpu.set_option("pair_l2_hint", hint)
            C = B.from_host(c0)
            gpu.gemm(B.from_host(a), B.from_host(b), C, trans_b=True, accumulate=True)
            torch.cuda.synchronize()
            outs.append(B.to_host(C))
    finally:
        gpu.set_option("pair_l2_hint", 3)
        gpu.set_option("force_path", 0)
    check(outs[0], orc.gemm(a, b, trans_b=True, c=c0, accumulate=True), np.float16)
    for o in outs[1:]:
        assert np.array_equal(o, outs[0])


def test_large_half_product_by_linearity(gpu):
    """C4 size (8192^3): (A*B)*v must equal A*(B*v).  Both sides are formed from fp16-rounded
    data with fp32 matrix-vector products, so the check is independent of any other GEMM."""
    n = 8192
    g = torch.Generator(device="cuda").manual_seed(5)
    A = torch.randn(n, n, device="cuda", generator=g).half().T
    Bm = torch.randn(n, n, device="cuda", generator=g).half().T
    dC = torch.randn(n, n, device="cuda", generator=g).half().T
    v = torch.randn(n, 1, device="cuda", generator=g, dtype=torch.float64)
    C = torch.empty(n, n, device="cuda", dtype=torch.float16).T
    gpu.gemm(A, Bm, C)
    lhs, rhs = C.double() @ v, A.double() @ (Bm.double() @ v)
    assert ((lhs - rhs).norm() / rhs.norm()).item() < 5e-3
    dA = torch.zeros(n, n, device="cuda", dtype=torch.float16).T
    gpu.gemm(dC, Bm, dA, trans_b=True, accumulate=True)
    lhs, rhs = dA.double() @ v, dC.double() @ (Bm.double().T @ v)
    assert ((lhs - rhs).norm() / rhs.norm()).item() < 5e-3
    dB = torch.zeros(n, n, device="cuda", dtype=torch.float16).T
    gpu.gemm(A, dC, dB, trans_a=True, accumulate=True)
    lhs, rhs = dB.double() @ v, A.double().T @ (dC.double() @ v)
    assert ((lhs - rhs).norm() / rhs.norm()).item() < 5e-3


def test_large_half_products_against_sampled_oracle(gpu):
    """C4 size (8192^3), all three products of the pass: 32 sampled rows x 64 sampled columns of
    every result against the fp64 oracle on exactly the operands the GPU used (the full fp64
    product would be hours of host time; a sampled block is a few GFLOP)."""
    n = 8192
    g = torch.Generator(device="cuda").manual_seed(6)
    A = torch.randn(n, n, device="cuda", generator=g).half().T
    Bm = torch.randn(n, n, device="cuda", generator=g).half().T
    dC = torch.randn(n, n, device="cuda", generator=g).half().T
    rs = np.random.default_rng(7)
    rows = torch.as_tensor(np.sort(rs.choice(n, 32, replace=False)), device="cuda")
    cols = torch.as_tensor(np.sort(rs.choice(n, 64, replace=False)), device="cuda")
    host = lambda t: t.cpu().numpy()
    out = torch.empty(n, n, device="cuda", dtype=torch.float16).T
    gpu.gemm(A, Bm, out)                                         # C = A B
    torch.cuda.synchronize()
    check(host(out[rows][:, cols]), orc.gemm(host(A[rows]), host(Bm[:, cols])), np.float16, "C")
    out.zero_()
    gpu.gemm(dC, Bm, out, trans_b=True, accumulate=True)         # dA += dC B^T
    torch.cuda.synchronize()
    check(host(out[rows][:, cols]), orc.gemm(host(dC[rows]), host(Bm[cols]), trans_b=True),
          np.float16, "dA")
    out.zero_()
    gpu.gemm(A, dC, out, trans_a=True, accumulate=True)          # dB += A^T dC
    torch.cuda.synchronize()
    check(host(out[rows][:, cols]), orc.gemm(host(A[:, rows]), host(dC[:, cols]), trans_a=True),
          np.float16, "dB")


def test_fp32_accuracy_holds_at_large_k(gpu):
    """dW of the MLP config contracts over the 4096-column batch."""
    rng = np.random.default_rng(18)
    for (m, n, k, ta, tb) in [(128, 96, 4096, False, True), (256, 128, 8192, False, False),
                              (160, 64, 20000, True, False), (96, 130, 17001, False, True)]:
        run_gemm(gpu, rng, np.float32, m, n, k, ta, tb, True)   # > 8192: chained launches
    run_gemm(gpu, rng, np.float32, 200, 72, 9000, False, False, False)


def test_assigning_products_with_split_contraction(gpu):
    """C = A*B (no accumulation) with few tiles and a long K: split over CTAs onto a zeroed C,
    also for a small strided batch and for a padded C whose padding must stay untouched."""
    rng = np.random.default_rng(24)
    run_gemm(gpu, rng, np.float32, 256, 128, 4096, False, False, False)
    run_gemm(gpu, rng, np.float32, 200, 100, 3000, True, False, False)
    a, b = randn(rng, (128, 1024, 3), np.float32), randn(rng, (1024, 128, 3), np.float32)
    C = B.colmajor(128, 128, torch.float32, batches=3, fill=5.0)
    gpu.gemm_batched(B.from_host(a), B.from_host(b), C)
    torch.cuda.synchronize()
    check(B.to_host(C), orc.gemm_batched(a, b), np.float32, "batched assign")
    a2, b2 = randn(rng, (128, 2048), np.float32), randn(rng, (2048, 64), np.float32)
    buf = B.colmajor(132, 64, torch.float32, fill=3.0)
    Cv = buf[:128]
    gpu.gemm(B.from_host(a2), B.from_host(b2), Cv)
    torch.cuda.synchronize()
    check(B.to_host(Cv), orc.gemm(a2, b2), np.float32, "padded assign")
    assert (B.to_host(buf)[128:] == 3.0).all()


def test_narrow_fp32_products(gpu):
    """Products with at most 64 rows or at most 64 columns (the attention backward's dV, dQ, dK'
    with a head of 64): the TMA kernel runs them on 128 x 64 tiles, the short-and-wide ones as the
    transposed product written through strides.  Every layout, assigning and adding, ragged
    extents, a padded C whose padding must survive, a long K (split) and a strided batch."""
    rng = np.random.default_rng(31)
    for (m, n, k) in [(64, 256, 128), (64, 128, 64), (48, 200, 96), (33, 1000, 260), (8, 136, 32),
                      (256, 64, 128), (200, 40, 96), (1000, 24, 260), (64, 640, 4096)]:
        for ta, tb in TRANS:
            run_gemm(gpu, rng, np.float32, m, n, k, ta, tb, False)
            run_gemm(gpu, rng, np.float32, m, n, k, ta, tb, True)
    for (m, n, k) in [(64, 256, 128), (40, 300, 72)]:
        a, b = randn(rng, (m, k), np.float32), randn(rng, (k, n), np.float32)
        buf = B.colmajor(m + 4, n, torch.float32, fill=3.0)
        Cv = buf[:m]
        gpu.gemm(B.from_host(a), B.from_host(b), Cv)
        torch.cuda.synchronize()
        check(B.to_host(Cv), orc.gemm(a, b), np.float32, "padded narrow")
        assert (B.to_host(buf)[m:] == 3.0).all()
    for acc in (False, True):
        a, b = randn(rng, (64, 128, 6), np.float32), randn(rng, (128, 256, 6), np.float32)
        c0 = randn(rng, (64, 256, 6), np.float32)
        C = B.from_host(c0)
        gpu.gemm_batched(B.from_host(a), B.from_host(b), C, accumulate=acc)
        torch.cuda.synchronize()
        ref = orc.gemm_batched(a, b, c=c0, accumulate=acc)
        check(B.to_host(C), ref, np.float32, f"batched narrow acc{acc}")


def test_short_contractions_with_more_tiles_than_sms(gpu):
    """fp32 products whose tiles have few k-blocks and outnumber the SMs: one CTA per SM walks the
    tiles (barriers and tensor memory set up once, accumulators handed back through a barrier).
    Ragged edges, every layout, assigning and adding, a strided batch, and the same product with
    the walk switched off."""
    rng = np.random.default_rng(35)
    for (m, n, k) in [(2000, 1500, 96), (1300, 2100, 40), (3000, 70, 200)]:
        for ta, tb in TRANS:
            run_gemm(gpu, rng, np.float32, m, n, k, ta, tb, False)
        run_gemm(gpu, rng, np.float32, m, n, k, False, False, True)
    a, b = randn(rng, (200, 100, 40), np.float32), randn(rng, (100, 150, 40), np.float32)
    c0 = randn(rng, (200, 150, 40), np.float32)
    for acc in (False, True):
        C = B.from_host(c0)
        gpu.gemm_batched(B.from_host(a), B.from_host(b), C, accumulate=acc)
        torch.cuda.synchronize()
        check(B.to_host(C), orc.gemm_batched(a, b, c=c0, accumulate=acc), np.float32, f"batched walk acc{acc}")
    gpu.set_option("walk_kblocks", 0)
    try:
        run_gemm(gpu, rng, np.float32, 2000, 1500, 96, False, False, True)
    finally:
        gpu.set_option("walk_kblocks", 16)


def test_non_finite_inputs_stay_where_they_belong(gpu):
    """An infinity in A and a NaN in B (fp32): exactly the row and the column of C they feed are
    non-finite, everything else matches the oracle (the hi/lo split must not leak inf - inf or a
    wrapped NaN pattern into other elements)."""
    rng = np.random.default_rng(33)
    for (m, n, k, ta, tb) in [(192, 160, 96, False, False), (130, 140, 70, True, False),
                              (64, 256, 128, False, True)]:
        a = randn(rng, (k, m) if ta else (m, k), np.float32)
        b = randn(rng, (n, k) if tb else (k, n), np.float32)
        if ta:
            a[5, 3] = np.inf
        else:
            a[3, 5] = np.inf
        nanbits = np.array([0xffffffff], np.uint32).view(np.float32)[0]
        if tb:
            b[2, 7] = nanbits
        else:
            b[7, 2] = nanbits
        C = B.colmajor(m, n, torch.float32, fill=0.0)
        gpu.gemm(B.from_host(a), B.from_host(b), C, ta, tb)
        torch.cuda.synchronize()
        got = B.to_host(C)
        bad = np.zeros((m, n), bool)
        bad[3, :] = True
        bad[:, 2] = True
        assert not np.isfinite(got[bad]).any()
        assert np.isnan(got[:, 2]).all()
        a0, b0 = np.where(np.isfinite(a), a, 0), np.where(np.isfinite(b), b, 0)
        ref = orc.gemm(a0, b0, ta, tb)
        np.testing.assert_allclose(got[~bad], ref[~bad], rtol=1e-4, atol=1e-4)


def test_empty_and_degenerate_shapes(gpu):
    rng = np.random.default_rng(19)
    c0 = randn(rng, (4, 5), np.float32)
    C = B.from_host(c0)
    a, b = B.colmajor(4, 0, torch.float32), B.colmajor(0, 5, torch.float32)
    gpu.gemm(a, b, C, accumulate=True)       # k == 0, Add: C unchanged
    torch.cuda.synchronize()
    np.testing.assert_array_equal(B.to_host(C), c0)
    gpu.gemm(a, b, C, accumulate=False)      # k == 0, Assign: C = 0
    torch.cuda.synchronize()
    assert not B.to_host(C).any()
    lib = gpu.lib()
    assert lib.ginn_b200_gemm(0, None, 0, 0, 0, 0, 5, 3, None, 1, None, 3, None, 1, 0) == 0  # m == 0


def test_argument_errors_are_reported(gpu):
    lib = gpu.lib()
    x = torch.zeros(16, device="cuda")
    p = x.data_ptr()
    assert lib.ginn_b200_gemm(0, None, 7, 0, 0, 2, 2, 2, p, 2, p, 2, p, 2, 0) == 2      # dtype
    assert lib.ginn_b200_gemm(0, None, 0, 0, 0, 4, 2, 2, p, 2, p, 2, p, 4, 0) == 1      # lda < m
    assert lib.ginn_b200_gemm(0, None, 0, 0, 0, -1, 2, 2, p, 2, p, 2, p, 2, 0) == 1     # negative
    assert lib.ginn_b200_gemm(0, None, 0, 0, 0, 2, 2, 2, None, 2, p, 2, p, 2, 0) == 1   # null
    assert b"null" in lib.ginn_b200_last_error()
    assert lib.ginn_b200_gemm(999, None, 0, 0, 0, 2, 2, 2, p, 2, p, 2, p, 2, 0) == 1    # device


def test_bounded_wait_reports_instead_of_hanging(gpu):
    """A wait that nothing answers must end by itself and leave its code in a status word; the
    context stays usable (the next product is correct) and the library's own status stays clean."""
    gpu.selftest(0)
    assert gpu.device_status(0, False) == 0
    run_gemm(gpu, np.random.default_rng(23), np.float32, 64, 48, 80, False, False, False)


@pytest.mark.parametrize("dt", [np.float32, np.float16])
def test_skinny_products_on_cuda_cores(gpu, dt):
    """One extent of at most 16 (config 5's ten-class output layer and its two gradients) or a
    contraction of at most 32: the CUDA-core mappings, every transpose, `=` and `+=`, batches,
    and the same shapes on the tensor-core path as a cross-check of the dispatch."""
    rng = np.random.default_rng(21)
    shapes = [(10, 4096, 1024), (1024, 512, 10), (10, 1024, 4096), (16, 300, 77), (3, 5, 2000),
              (200, 300, 7), (1, 513, 640), (7, 129, 33),
              # the streaming variants' edges: ragged column groups, K not a multiple of the
              # vector, row blocks beyond 1024, a contraction between 17 and 32
              (12, 600, 516), (10, 1000, 4096), (16, 132, 640), (2048, 300, 12), (1028, 70, 25)]
    for (m, n, k) in shapes:
        for ta, tb in TRANS:
            for acc in (False, True):
                run_gemm(gpu, rng, dt, m, n, k, ta, tb, acc)
    run_gemm(gpu, rng, dt, 10, 333, 129, False, True, True, 3, 1)  # padded, unaligned, NT +=
    run_gemm(gpu, rng, dt, 10, 1024, 2048, False, True, True, 2, 0)  # padded C: scalar atomics
    run_gemm(gpu, rng, dt, 1024, 256, 10, True, False, True, 4, 0)   # padded C, aligned
    a, b = randn(rng, (10, 96, 6), dt), randn(rng, (96, 200, 6), dt)
    c0 = randn(rng, (10, 200, 6), dt)
    for acc in (False, True):
        C = B.from_host(c0)
        gpu.gemm_batched(B.from_host(a), B.from_host(b), C, False, False, acc)
        torch.cuda.synchronize()
        check(B.to_host(C), orc.gemm_batched(a, b, False, False, c0, acc), dt, "batched skinny")
    launches = gpu.launch_count()
    run_gemm(gpu, rng, dt, 10, 4096, 1024, False, False, False)
    assert gpu.launch_count() == launches + 1


@pytest.mark.parametrize("dt", [np.float32, np.float16])
def test_prod_backward_in_one_call(gpu, dt):
    """ProdNode::backward_ and BatchedProdNode::backward_ (ginn/node/prod.h:51-66, 118-130) as
    one entry: da += dc b^T and db += a^T dc, run side by side by the library; either gradient
    alone; the option that keeps them on one stream; and Prod(x, x), whose two gradients are one
    tensor and therefore must not run side by side."""
    rng = np.random.default_rng(29)
    for (m, n, k) in [(3, 2, 5), (200, 96, 130), (512, 768, 256), (1024, 1024, 1024)]:
        a, b, dc = randn(rng, (m, k), dt), randn(rng, (k, n), dt), randn(rng, (m, n), dt)
        da0, db0 = randn(rng, (m, k), dt), randn(rng, (k, n), dt)
        rda = orc.gemm(dc, b, trans_b=True, c=da0, accumulate=True)
        rdb = orc.gemm(a, dc, trans_a=True, c=db0, accumulate=True)
        for fork in (1, 0):
            gpu.set_option("fork_streams", fork)
            try:
                A, Bm, dC, dA, dB = map(B.from_host, (a, b, dc, da0, db0))
                gpu.prod_backward(A, Bm, dC, dA, dB)
                torch.cuda.synchronize()
            finally:
                gpu.set_option("fork_streams", 1)
            check(B.to_host(dA), rda, dt, f"da {m} {n} {k} fork{fork}")
            check(B.to_host(dB), rdb, dt, f"db {m} {n} {k} fork{fork}")
        dA, dB = B.from_host(da0), B.from_host(db0)
        gpu.prod_backward(B.from_host(a), B.from_host(b), B.from_host(dc), dA, None)
        gpu.prod_backward(B.from_host(a), B.from_host(b), B.from_host(dc), None, dB)
        torch.cuda.synchronize()
        check(B.to_host(dA), rda, dt, "da alone")
        check(B.to_host(dB), rdb, dt, "db alone")
    # c = x x with x square: both gradients accumulate into x's one gradient tensor
    x, dc, g0 = randn(rng, (256, 256), dt), randn(rng, (256, 256), dt), randn(rng, (256, 256), dt)
    X, G = B.from_host(x), B.from_host(g0)
    gpu.prod_backward(X, X, B.from_host(dc), G, G)
    torch.cuda.synchronize()
    ref = orc.gemm(dc, x, trans_b=True, c=g0, accumulate=True)
    if dt == np.float16:  # the library rounds to fp16 between the two additions
        ref = ref.astype(np.float16)
    ref = orc.gemm(x, dc, trans_a=True, c=ref, accumulate=True)
    check(B.to_host(G), ref, dt, "Prod(x, x)")
    # batched, rank 3
    a, b, dc = randn(rng, (64, 48, 7), dt), randn(rng, (48, 80, 7), dt), randn(rng, (64, 80, 7), dt)
    dA = B.colmajor(64, 48, torch.from_numpy(a[:1, :1, 0]).dtype, batches=7, fill=0.0)
    dB = B.colmajor(48, 80, torch.from_numpy(a[:1, :1, 0]).dtype, batches=7, fill=0.0)
    gpu.prod_backward(B.from_host(a), B.from_host(b), B.from_host(dc), dA, dB)
    torch.cuda.synchronize()
    check(B.to_host(dA), orc.gemm_batched(dc, b, trans_b=True), dt, "batched da")
    check(B.to_host(dB), orc.gemm_batched(a, dc, trans_a=True), dt, "batched db")


def test_large_fp32_products_with_operands_split_once(gpu):
    """Products with at least four tiles along both extents and a full wave of tiles split their
    operands into hi / lo planes once, in a scratch allocation, and run on a kernel that TMA feeds
    directly.  Every transpose form, accumulation, ragged extents with a contraction that is not
    a multiple of 32, padded leading dimensions, and the same products with the option off."""
    rng = np.random.default_rng(31)
    for (m, n, k) in [(1024, 4096, 1024), (1500, 2100, 300), (2048, 1300, 2050)]:
        for ta, tb in TRANS:
            for acc in (False, True):
                got, ref = run_gemm(gpu, rng, np.float32, m, n, k, ta, tb, acc)
    run_gemm(gpu, rng, np.float32, 1100, 2200, 516, False, True, True, ld_pad=4, offset=8)
    # few tiles and a long contraction: the split-once kernel with the contraction split over CTAs
    for ta, tb in TRANS:
        for acc in (False, True):
            run_gemm(gpu, rng, np.float32, 1024, 784, 4100, ta, tb, acc)
    # same answers (to rounding) without the split-once path
    a, b = randn(rng, (1536, 640), np.float32), randn(rng, (640, 2048), np.float32)
    outs = []
    try:
        for on in (1, 0):
            gpu.set_option("presplit", on)
            C = B.colmajor(1536, 2048, torch.float32, fill=0.0)
            gpu.gemm(B.from_host(a), B.from_host(b), C)
            torch.cuda.synchronize()
            outs.append(B.to_host(C))
    finally:
        gpu.set_option("presplit", 1)
    check(outs[0], orc.gemm(a, b), np.float32)
    check_elementwise(outs[0], orc.gemm(a, b), np.float32)
    assert np.abs(outs[0] - outs[1]).max() <= 1e-5 * np.abs(outs[1]).max()
