"""Base class of the GEMM + all-scatter overlap patterns."""

from __future__ import annotations

import abc
from typing import Any, Optional

from .contracts import PatternExecutionSpec, resolve_pattern_execution


class Pattern(abc.ABC):
    """One way of overlapping ``C = A @ B`` with pushing column slices to the peers.

    Subclasses set ``name`` and implement ``_run(A, B, C, spec)``.  Constructor
    keyword arguments of the reference's patterns (``BLOCK_M``, ``NUM_SMS``,
    ``COMM_SMS`` ..., tileccl/patterns/wg_specialized.py:66-80) are accepted and
    recorded; the tile shape of the sm_100a kernel is fixed at 128 x 256 x 64.
    """

    name: str = "base"

    def __init__(self, ctx: Any, **options: Any) -> None:
        self.ctx = ctx
        self.options = dict(options)

    # ---------------------------------------------------------------- contract
    def resolve_execution(self, A, B, C, *, spec: Optional[PatternExecutionSpec] = None,
                          full_N: Optional[int] = None, b_layout: Optional[str] = None,
                          c_layout: Optional[str] = None,
                          storage_kind: str = "symmetric") -> PatternExecutionSpec:
        if spec is not None:
            return spec
        return resolve_pattern_execution(A, B, C, rank=self.ctx.rank,
                                         world_size=self.ctx.world_size, full_N=full_N,
                                         b_layout=b_layout, c_layout=c_layout,
                                         storage_kind=storage_kind)

    def require_device_remote_access_runtime(self, *, operation: str) -> None:
        """Raise unless the context's heap lets device code reach every peer."""
        if self.ctx.world_size == 1:
            return
        heap = self.ctx.require_heap()
        from ..utils.feature_gates import (multiprocess_device_remote_access_detail,
                                           multiprocess_device_remote_access_transport_supported)

        if heap.mode == "multiprocess" and not multiprocess_device_remote_access_transport_supported(
                heap.transport_strategy):
            raise ValueError(multiprocess_device_remote_access_detail(
                transport_strategy=heap.transport_strategy, operation=operation))

    # --------------------------------------------------------------- execution
    def execute(self, A, B, C, **kwargs: Any) -> None:
        spec = self.resolve_execution(A, B, C, **kwargs)
        self.require_device_remote_access_runtime(operation=f"{self.name}.execute")
        self._run(A, B, C, spec)

    @abc.abstractmethod
    def _run(self, A, B, C, spec: PatternExecutionSpec) -> None:
        ...

    def benchmark(self, A, B, C, warmup: int = 10, iters: int = 100, **execute_kwargs: Any) -> dict:
        """Device-timed (CUDA events) latency of ``execute``."""
        import torch

        for _ in range(warmup):
            self.execute(A, B, C, **execute_kwargs)
        torch.cuda.synchronize(A.device)
        times = []
        for _ in range(iters):
            s = torch.cuda.Event(enable_timing=True)
            e = torch.cuda.Event(enable_timing=True)
            s.record()
            self.execute(A, B, C, **execute_kwargs)
            e.record()
            e.synchronize()
            times.append(s.elapsed_time(e))
        return {"pattern": self.name, "mean_ms": sum(times) / len(times), "min_ms": min(times),
                "max_ms": max(times), "iters": iters, "timing": "cuda_events"}

    def __repr__(self) -> str:
        return f"{type(self).__name__}(rank={self.ctx.rank}/{self.ctx.world_size})"
