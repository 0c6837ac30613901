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
    """One forward+backward pass of ProdNode (ginn/node/prod.h:28-66) on a column shard.

    `panels` > 1 splits dA = dC * B^T into that many column panels of dA (row blocks of the
    local B shard, i.e. pointer offsets into column-major storage, no copy): the reduction of a
    finished panel starts while the later panels and the dB product are still being computed,
    so only the last panel's reduction is exposed.  `col_block(x, first, count)` must return the
    view of columns [first, first+count) of x, `row_block` the same for rows.
    """

    def __init__(self, gemm: Callable, zero: Callable, allreduce_async: Callable, panels: int = 1,
                 col_block: Callable = None, row_block: Callable = None,
                 overlapped: Callable = None, zero_beside: Callable = None):
        self.gemm = gemm
        self.zero = zero
        # optional: zero_beside([tensors]) clears the gradients off the main stream (they are
        # first touched by the second product) and returns the function that waits for it
        self.zero_beside = zero_beside
        self.allreduce_async = allreduce_async
        self.panels = max(1, panels)
        self.col_block = col_block or (lambda x, s, c: x[:, s:s + c])
        self.row_block = row_block or (lambda x, s, c: x[s:s + c])
        # called with True before the first product that runs beside a reduction and with
        # False after the last one (the GPU harness reserves SMs for the collective there)
        self.overlapped = overlapped or (lambda on: None)

    def step(self, A, B_shard, dC_shard, C_shard, dA, dB_shard, between: Callable = None):
        """C = A*B; dA += dC*B^T (all-reduced); dB += A^T*dC.  Gradients are zeroed first, as
        Graph::reset_grad does.  `between(i)` is called after product i (timing hooks)."""
        zeroed = None
        if self.zero_beside is not None:
            zeroed = self.zero_beside([dA, dB_shard])   # runs beside the forward product
        else:
            self.zero(dA)
            self.zero(dB_shard)
        self.gemm(A, B_shard, C_shard, False, False, False)
        if zeroed is not None:
            zeroed()
        if between:
            between(0)
        waits = []
        k = dA.shape[1]
        for p in range(self.panels):
            s, c = column_shard(k, self.panels, p)
            if c == 0:
                continue
            if waits:
                self.overlapped(True)
            # columns [s, s+c) of dA = dC * (rows [s, s+c) of B)^T
            self.gemm(dC_shard, self.row_block(B_shard, s, c), self.col_block(dA, s, c), False,
                      True, True)
            waits.append(self.allreduce_async(self.col_block(dA, s, c)))
        if between:
            between(1)
        self.overlapped(True)
        self.gemm(A, dC_shard, dB_shard, True, False, True)
        self.overlapped(False)
        if between:
            between(2)
        for w in waits:
            w()
