"""Chained all-gather -> GEMM -> reduce-scatter pattern.

The reference's kernel of this name gathers a K-sharded operand, multiplies, and
then copies whole output tiles to every peer without reducing them
(tileccl/patterns/chained_ag_gemm_rs.py:201-425).  Here the chain has the intended
meaning: the row-sharded operand is gathered by the GEMM kernel itself, and a
second GEMM reduce-scatters its partial sums (``parallel.chain`` /
``ops._fused.reduce_scatter``)."""

from ..ops import _fused
from ..parallel.chain import rows_allgather_gemm
from .base import Pattern


class ChainedAGGemmRSPattern(Pattern):
    name = "chained_ag_gemm_rs"

    def run_chain(self, x_full, W1, hidden, W2, out_local, *, epilogue: str = "none"):
        """``out_local = reduce_scatter_rows(epilogue(allgather_rows(x) @ W1) @ W2)``."""
        rows_allgather_gemm(self.ctx, self.name + ":ag", x_full, W1, hidden, epilogue=epilogue)
        _fused.reduce_scatter(self.ctx, self.name + ":rs", hidden, W2, out_local, split_axis=0)
        return out_local

    def _run(self, A, B, C, spec) -> None:
        raise NotImplementedError(
            "ChainedAGGemmRSPattern is driven through run_chain(x_full, W1, hidden, W2, out_local)")
