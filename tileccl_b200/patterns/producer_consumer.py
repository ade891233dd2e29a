"""Producer / consumer pattern: the GEMM kernel publishes every finished band of
128 rows on a counter; a push kernel on a second stream sends a band to the peers
as soon as its counter is complete (reference:
tileccl/patterns/producer_consumer.py:245-393, per-tile locks there)."""

from .base import Pattern
from ._impl import run_two_kernel


class ProducerConsumerPattern(Pattern):
    name = "producer_consumer"
    split = "kernels"

    def _run(self, A, B, C, spec) -> None:
        run_two_kernel(self.ctx, self.name, A, B, C, spec, overlapped=True,
                       shape=self.launch_shape())
