"""Fused-sequential pattern: one kernel; the warps that convert a tile also store it
to the local output and to every peer with 16-byte stores, tile after tile
(reference: tileccl/patterns/fused_sequential.py:145-254)."""

from ..kernels import fused_gemm as fg
from .base import Pattern
from ._impl import pick_push_mode, run_fused


class FusedSequentialPattern(Pattern):
    name = "fused_sequential"

    def _run(self, A, B, C, spec) -> None:
        run_fused(self.ctx, self.name, A, B, C, spec, pick_push_mode(self.ctx, fg.PUSH_STORES),
                  shape=self.launch_shape())
