"""Bulk-synchronous pattern: whole GEMM first, then one push of the column slice.

Two launches in stream order (reference: tileccl/patterns/bulk_sync.py:160-299,
which separates them with a host synchronisation)."""

from .base import Pattern
from ._impl import run_two_kernel


class BulkSyncPattern(Pattern):
    name = "bulk_sync"
    split = "kernels"

    def _run(self, A, B, C, spec) -> None:
        run_two_kernel(self.ctx, self.name, A, B, C, spec, overlapped=False,
                       shape=self.launch_shape())
