"""Column sharding of the Prod path over ranks (one process per GPU).

For C = A*B with ginn's column = batch convention (ginn/node/layout.h:219-220) the natural split
is over the columns of B, C and dC; A is replicated.  Forward and dB = A^T*dC then need no
exchange.  dA = dC*B^T sums over the sharded columns, so every rank's contribution is all-reduced;
the reduction is issued as soon as dA is produced and overlaps the dB product.

The class is backend-agnostic: `gemm` is the product routine (the C ABI on a GPU; the tests use
the CPU oracle with the gloo backend), `allreduce_async` starts the reduction and returns a
callable that waits for it.
"""
from __future__ import annotations

from typing import Callable, Tuple


def column_shard(n_total: int, world: int, rank: int) -> Tuple[int, int]:
    """First column and column count of `rank`'s shard (remainder spread over the low ranks)."""
    base, rem = divmod(n_total, world)
    count = base + (1 if rank < rem else 0)
    start = rank * base + min(rank, rem)
    return start, count


class ShardedProd:
    """One forward+backward pass of ProdNode (ginn/node/prod.h:28-66) on a column shard."""

    def __init__(self, gemm: Callable, zero: Callable, allreduce_async: Callable):
        self.gemm = gemm
        self.zero = zero
        self.allreduce_async = allreduce_async

    def step(self, A, B_shard, dC_shard, C_shard, dA, dB_shard, between: Callable = None):
        """C = A*B; dA += dC*B^T (all-reduced); dB += A^T*dC.  Gradients are zeroed first, as
        Graph::reset_grad does.  `between(i)` is called after product i (timing hooks)."""
        self.zero(dA)
        self.zero(dB_shard)
        self.gemm(A, B_shard, C_shard, False, False, False)
        if between:
            between(0)
        self.gemm(dC_shard, B_shard, dA, False, True, True)
        if between:
            between(1)
        wait = self.allreduce_async(dA)
        self.gemm(A, dC_shard, dB_shard, True, False, True)
        if between:
            between(2)
        wait()
