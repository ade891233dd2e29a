"""Base class of the GEMM + all-scatter overlap patterns."""

from __future__ import annotations

import abc
from typing import Any, Optional

from .contracts import PatternExecutionSpec, resolve_pattern_execution


class Pattern(abc.ABC):
    """One way of overlapping ``C = A @ B`` with pushing column slices to the peers.

    Subclasses set ``name``, ``split`` and implement ``_run(A, B, C, spec)``.

    Constructor keyword arguments follow the reference's patterns
    (tileccl/patterns/wg_specialized.py:66-80):

    * ``NUM_SMS`` / ``COMPUTE_SMS``: CTAs of the GEMM launch (default: every SM);
    * ``COMM_SMS``: CTAs of the communication role.  The two-kernel patterns
      (``split = "kernels"``: bulk_sync, producer_consumer) launch their push kernel on that
      many CTAs.  In the single-kernel patterns (``split = "warps"``) the communication role
      is played by warps inside every compute CTA, so an SM split cannot be honoured and
      ``COMM_SMS > 0`` is rejected with an error instead of being ignored;
    * ``BLOCK_M / BLOCK_N / BLOCK_K``: the tcgen05 tile is fixed at 128 x 256 x 64 (256 x 256
      per CTA pair); other values are rejected unless they are the reference's own defaults
      (128 x 128 x 64), which are taken to mean "default".

    ``launch_shape()`` returns the resolved split (a ``DualRoleScheduler``).
    """

    name: str = "base"
    split: str = "warps"         # "warps": comm role = warps of each CTA; "kernels": own launch

    def __init__(self, ctx: Any, **options: Any) -> None:
        self.ctx = ctx
        self.options = dict(options)
        unknown = set(options) - {"BLOCK_M", "BLOCK_N", "BLOCK_K", "NUM_SMS", "COMPUTE_SMS",
                                  "COMM_SMS", "num_warps", "num_stages", "GROUP_SIZE_M"}
        if unknown:
            raise TypeError(f"{type(self).__name__} got unexpected options {sorted(unknown)}")
        tile = (options.get("BLOCK_M", 128), options.get("BLOCK_N", 128), options.get("BLOCK_K", 64))
        if tile not in ((128, 128, 64), (128, 256, 64)):
            raise ValueError(f"the sm_100a kernel works on 128 x 256 x 64 tiles; BLOCK_M/N/K = {tile} "
                             "cannot be honoured")
        comm = int(options.get("COMM_SMS", 0) or 0)
        if comm < 0:
            raise ValueError("COMM_SMS must be non-negative")
        if comm and self.split == "warps":
            raise ValueError(
                f"{self.name}: communication runs on warps inside every compute CTA of the fused "
                "kernel, so COMM_SMS cannot set SMs aside; use producer_consumer or bulk_sync "
                "for an SM split, or drop COMM_SMS")

    def launch_shape(self):
        """How many CTAs compute and how many communicate (resolved against the device)."""
        from .runtime import B200_SMS

        total = B200_SMS
        try:
            props = self.ctx.backend.get_device_properties(0) if self.ctx.backend else None
            total = props.compute_units if props is not None else B200_SMS
        except Exception:
            total = B200_SMS
        total = int(self.options.get("NUM_SMS", total) or total)
        compute = int(self.options.get("COMPUTE_SMS", 0) or 0)
        comm = int(self.options.get("COMM_SMS", 0) or 0)
        if self.split == "kernels":
            # Two launches: each gets its own grid; they may add up to more than the device
            # has (the push kernel's CTAs are small and co-reside with the GEMM's).
            from .runtime import DEFAULT_PUSH_GRID, DualRoleScheduler

            return DualRoleScheduler(total, compute or total, comm or DEFAULT_PUSH_GRID,
                                     comm_warps_per_cta=16, policy="two_kernels")
        from .runtime import DualRoleScheduler

        # warps of every compute CTA communicate: SMs that do not compute stay idle
        return DualRoleScheduler(total, min(compute or total, total), 0, policy="in_cta_comm_warps")

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
