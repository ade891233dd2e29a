"""Overlap patterns for GEMM + all-scatter (``ops.gemm_allscatter(pattern=...)``).

Names and aliases follow the reference (tileccl/patterns/__init__.py:192-214,
tileccl/ops.py:74-83)."""

from __future__ import annotations

from typing import Any, Optional

from .base import Pattern
from .bulk_sync import BulkSyncPattern
from .chained_ag_gemm_rs import ChainedAGGemmRSPattern
from .contracts import (PatternExecutionSpec, PatternTensorSpec, resolve_pattern_execution,
                        spec_from_contract)
from .fused_sequential import FusedSequentialPattern
from .producer_consumer import ProducerConsumerPattern
from .runtime import (DualRoleScheduler, StageRoleScheduler, TileCollectiveExecution,
                      TileCollectiveRuntime, resolve_dual_role_scheduler,
                      resolve_stage_role_scheduler, resolve_tile_collective_execution,
                      resolve_tile_collective_runtime)
from .wg_specialized import WGSpecializedPattern

PATTERN_CLASSES = {
    "bulk_sync": BulkSyncPattern,
    "fused_sequential": FusedSequentialPattern,
    "producer_consumer": ProducerConsumerPattern,
    "wg_specialized": WGSpecializedPattern,
}
PATTERN_ALIASES = {"auto": None, "fused_seq": "fused_sequential", "pc": "producer_consumer",
                   "wg_spec": "wg_specialized", **{k: k for k in PATTERN_CLASSES}}

from .auto_select import auto_select, benchmark_all_patterns  # noqa: E402


def resolve_pattern(pattern: Any, *, ctx, M: int, N: int, K: int, hw_info: Any = None) -> Pattern:
    """``pattern`` may be a name / alias, ``None`` / "auto", a Pattern subclass or an instance."""
    if isinstance(pattern, Pattern):
        return pattern
    if isinstance(pattern, type) and issubclass(pattern, Pattern):
        return pattern(ctx)
    if pattern is None:
        pattern = "auto"
    if not isinstance(pattern, str) or pattern not in PATTERN_ALIASES:
        raise ValueError(f"unknown pattern {pattern!r}; expected one of {sorted(PATTERN_ALIASES)}")
    name = PATTERN_ALIASES[pattern]
    if name is None:
        return auto_select("gemm_allscatter", M, N, K, world_size=ctx.world_size, ctx=ctx,
                           hw_info=hw_info)
    return PATTERN_CLASSES[name](ctx)


__all__ = ["Pattern", "BulkSyncPattern", "FusedSequentialPattern", "ProducerConsumerPattern",
           "WGSpecializedPattern", "ChainedAGGemmRSPattern", "PatternExecutionSpec",
           "PatternTensorSpec", "resolve_pattern_execution", "spec_from_contract",
           "DualRoleScheduler", "StageRoleScheduler", "TileCollectiveExecution",
           "TileCollectiveRuntime", "resolve_dual_role_scheduler", "resolve_stage_role_scheduler",
           "resolve_tile_collective_execution", "resolve_tile_collective_runtime", "auto_select",
           "benchmark_all_patterns", "resolve_pattern", "PATTERN_CLASSES", "PATTERN_ALIASES"]
