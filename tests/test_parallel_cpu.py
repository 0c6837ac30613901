"""world_size-2 test of the column-sharded Prod path on CPU (gloo), with the oracle standing in
for the GPU products: the sharded pass must reproduce the unsharded one."""
import os

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from ginn_b200.parallel import ShardedProd, column_shard
from oracle import oracle as orc


def test_column_shard_covers_everything():
    for n, w in [(10, 3), (8192, 8), (5, 8), (7, 1)]:
        cols = []
        for r in range(w):
            s, c = column_shard(n, w, r)
            cols += list(range(s, s + c))
        assert cols == list(range(n))


def _worker(rank, world, port, q, panels=1):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    rng = np.random.default_rng(3)                      # same stream on every rank: global data
    m, k, n = 24, 20, 30
    A = rng.standard_normal((m, k)).astype(np.float32)
    Bf = rng.standard_normal((k, n)).astype(np.float32)
    dCf = rng.standard_normal((m, n)).astype(np.float32)
    s, c = column_shard(n, world, rank)
    Bs, dCs = Bf[:, s:s + c], dCf[:, s:s + c]

    def gemm(a, b, out, ta, tb, acc):
        out[...] = orc.gemm(a, b, ta, tb, out, acc).astype(np.float32)

    def zero(x):
        x[...] = 0

    def allreduce_async(x):
        t = torch.from_numpy(np.ascontiguousarray(x))   # a column panel is a strided view here
        work = dist.all_reduce(t, async_op=True)

        def wait():
            work.wait()
            x[...] = t.numpy()
        return wait

    C = np.empty((m, c), np.float32)
    dA = np.full((m, k), 7.0, np.float32)               # stale values must be zeroed by the step
    dB = np.full((k, c), 7.0, np.float32)
    ShardedProd(gemm, zero, allreduce_async, panels=panels).step(A, Bs, dCs, C, dA, dB)
    ok = (np.allclose(C, A @ Bs, rtol=1e-5, atol=1e-5)
          and np.allclose(dA, dCf @ Bf.T, rtol=1e-4, atol=1e-4)
          and np.allclose(dB, A.T @ dCs, rtol=1e-5, atol=1e-5))
    q.put((rank, bool(ok)))
    dist.destroy_process_group()


@pytest.mark.parametrize("panels", [1, 3])
def test_sharded_prod_matches_unsharded_on_two_ranks(panels):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + (os.getpid() + 7 * panels) % 2000
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q, panels)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    assert sorted(results) == [(0, True), (1, True)]


def test_gradients_cleared_beside_the_forward_product():
    """`zero_beside` replaces the two `zero` calls: it is handed both gradients before the
    forward product, and its waiter runs before the first product that adds to them."""
    rng = np.random.default_rng(5)
    m, k, n = 12, 9, 14
    A = rng.standard_normal((m, k)).astype(np.float32)
    Bm = rng.standard_normal((k, n)).astype(np.float32)
    dC = rng.standard_normal((m, n)).astype(np.float32)
    events, pending = [], []

    def gemm(a, b, out, ta, tb, acc):
        events.append("add" if acc else "assign")
        out[...] = orc.gemm(a, b, ta, tb, out, acc).astype(np.float32)

    def zero(x):
        raise AssertionError("zero() must not be called when zero_beside is given")

    def zero_beside(ts):
        events.append("fork")
        pending.extend(ts)                 # cleared only when the waiter runs, as on a second stream

        def wait():
            events.append("join")
            for t in pending:
                t[...] = 0
        return wait

    C = np.empty((m, n), np.float32)
    dA = np.full((m, k), 3.0, np.float32)
    dB = np.full((k, n), 3.0, np.float32)
    ShardedProd(gemm, zero, lambda x: (lambda: None), panels=2, zero_beside=zero_beside).step(
        A, Bm, dC, C, dA, dB)
    assert events[:3] == ["fork", "assign", "join"] and events[3:] == ["add", "add", "add"]
    assert np.allclose(C, A @ Bm, rtol=1e-5, atol=1e-5)
    assert np.allclose(dA, dC @ Bm.T, rtol=1e-4, atol=1e-4)
    assert np.allclose(dB, A.T @ dC, rtol=1e-5, atol=1e-5)
