"""Warp-specialised pattern: one persistent kernel whose roles run concurrently -
TMA producer warp, tcgen05 issuer warp, and epilogue warps that hand every finished
tile to the TMA engine as bulk stores to the local output and to each peer, then
signal the TileGroup one tile later so the NVLink round trip overlaps the next
tile (reference: tileccl/patterns/wg_specialized.py:210-352, where whole SMs take
the communication role)."""

from ..kernels import fused_gemm as fg
from .base import Pattern
from ._impl import pick_push_mode, run_fused


class WGSpecializedPattern(Pattern):
    name = "wg_specialized"

    def _run(self, A, B, C, spec) -> None:
        run_fused(self.ctx, self.name, A, B, C, spec, pick_push_mode(self.ctx, fg.PUSH_TMA),
                  shape=self.launch_shape())
