"""Role split and collective-runtime metadata of the overlap patterns.

The reference divides *SMs* between a compute role and a communication role
(tileccl/patterns/runtime.py:108-383; 20 % of the SMs move data).  On B200 the
fused kernel keeps every SM on the tensor cores and gives the communication role
to warps inside each CTA (four epilogue warps, plus one warp that pushes the
all-gathered operand), so the default split here is ``comm_sms = 0`` with
``comm_warps_per_cta = 4``.  The two-kernel patterns still use an SM split: the
region-push kernel runs on a small grid next to the persistent GEMM.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Union

B200_SMS = 148
DEFAULT_COMM_WARPS_PER_CTA = 4
DEFAULT_PUSH_GRID = 32


@dataclass(frozen=True)
class DualRoleScheduler:
    total_sms: int
    compute_sms: int
    comm_sms: int
    comm_warps_per_cta: int = DEFAULT_COMM_WARPS_PER_CTA
    policy: str = "in_cta_comm_warps"

    def to_dict(self) -> dict:
        return dict(self.__dict__)


@dataclass(frozen=True)
class StageRoleScheduler:
    total_sms: int
    gather_sms: int
    compute_sms: int
    scatter_sms: int
    gather_warps_per_cta: int = 1
    scatter_warps_per_cta: int = DEFAULT_COMM_WARPS_PER_CTA
    policy: str = "in_cta_stage_warps"

    def to_dict(self) -> dict:
        return dict(self.__dict__)


@dataclass(frozen=True)
class TileCollectiveRuntime:
    op: str
    kernel: str
    signal_mode: str = "counting"
    wait_mode: str = "wait_ge"
    flow_control: str = "epoch_parity_double_buffer"
    transport: str = "peer_store"

    def to_dict(self) -> dict:
        return dict(self.__dict__)


@dataclass(frozen=True)
class TileCollectiveExecution:
    runtime: TileCollectiveRuntime = field(repr=False)
    scheduler: Union[DualRoleScheduler, StageRoleScheduler] = field(repr=False)
    queue_name: str = ""
    slot_count: int = 1
    credit_window: int = 1
    tile_rows: int = 128
    workspace_owners: tuple = ()
    queue_policy: str = "tilegroup_counters"

    def __post_init__(self) -> None:
        if self.slot_count < 1 or self.credit_window < 1 or self.tile_rows < 1:
            raise ValueError("slot_count, credit_window and tile_rows must be positive")

    def slot_workspace_names(self, slot_index: int) -> tuple:
        if not 0 <= slot_index < self.slot_count:
            raise ValueError(f"slot_index {slot_index} out of range for {self.slot_count} slots")
        return tuple(f"{self.queue_name}.{owner}.slot{slot_index}" for owner in self.workspace_owners)

    def to_dict(self) -> dict:
        return {"runtime": self.runtime.to_dict(), "scheduler": self.scheduler.to_dict(),
                "queue_name": self.queue_name, "slot_count": self.slot_count,
                "credit_window": self.credit_window, "tile_rows": self.tile_rows,
                "workspace_owners": list(self.workspace_owners), "queue_policy": self.queue_policy}


def resolve_dual_role_scheduler(total_sms: int, *, compute_sms: int = 0, comm_sms: int = 0,
                                comm_sm_fraction: float = 0.0) -> DualRoleScheduler:
    """Explicit counts win; otherwise ``comm_sm_fraction`` of the SMs communicate
    (default 0: communication runs on warps inside the compute CTAs)."""
    if total_sms <= 0:
        raise ValueError("total_sms must be positive")
    if compute_sms < 0 or comm_sms < 0:
        raise ValueError("SM counts must be non-negative")
    if compute_sms and comm_sms:
        if compute_sms + comm_sms > total_sms:
            raise ValueError(f"compute_sms + comm_sms = {compute_sms + comm_sms} exceeds {total_sms}")
        return DualRoleScheduler(total_sms, compute_sms, comm_sms, policy="explicit")
    if comm_sms:
        comm = comm_sms
    elif compute_sms:
        comm = total_sms - compute_sms
    else:
        comm = int(total_sms * comm_sm_fraction)
    comm = min(max(comm, 0), total_sms - 1)
    policy = "in_cta_comm_warps" if comm == 0 else "sm_split"
    return DualRoleScheduler(total_sms, total_sms - comm, comm, policy=policy)


def resolve_stage_role_scheduler(total_sms: int, *, gather_sms: int = 0, compute_sms: int = 0,
                                 scatter_sms: int = 0,
                                 collective_sm_fraction: float = 0.0) -> StageRoleScheduler:
    if total_sms <= 0:
        raise ValueError("total_sms must be positive")
    if min(gather_sms, compute_sms, scatter_sms) < 0:
        raise ValueError("SM counts must be non-negative")
    if gather_sms or scatter_sms or compute_sms:
        used = gather_sms + scatter_sms
        comp = compute_sms or total_sms - used
        if comp < 1 or used + comp > total_sms:
            raise ValueError("stage SM counts do not fit the device")
        return StageRoleScheduler(total_sms, gather_sms, comp, scatter_sms, policy="explicit")
    each = int(total_sms * collective_sm_fraction / 2)
    return StageRoleScheduler(total_sms, each, total_sms - 2 * each, each,
                              policy="in_cta_stage_warps" if each == 0 else "sm_split")


_RUNTIMES = {
    "gemm_allgather": TileCollectiveRuntime("gemm_allgather", "fused_gemm_sm100/push_all"),
    "gemm_reducescatter": TileCollectiveRuntime("gemm_reducescatter",
                                                "fused_gemm_sm100/reduce_scatter"),
    "allgather_gemm_reducescatter": TileCollectiveRuntime(
        "allgather_gemm_reducescatter", "fused_gemm_sm100/ag_push + reduce_scatter",
        flow_control="arrival_counters"),
    "gemm_allscatter": TileCollectiveRuntime("gemm_allscatter", "fused_gemm_sm100/all_scatter",
                                             flow_control="none"),
}


def resolve_tile_collective_runtime(op: str) -> TileCollectiveRuntime:
    try:
        return _RUNTIMES[op]
    except KeyError:
        raise ValueError(f"unknown tile-collective op {op!r}; expected one of {sorted(_RUNTIMES)}") from None


def resolve_tile_collective_execution(op: str, *, total_sms: int, rows: int, world_size: int,
                                      tile_rows: int = 128,
                                      max_groups: int = 64) -> TileCollectiveExecution:
    runtime = resolve_tile_collective_runtime(op)
    if rows <= 0 or world_size <= 0:
        raise ValueError("rows and world_size must be positive")
    if op == "allgather_gemm_reducescatter":
        scheduler = resolve_stage_role_scheduler(total_sms)
    else:
        scheduler = resolve_dual_role_scheduler(total_sms)
    bands = -(-rows // tile_rows)
    slots = min(bands, max_groups)
    return TileCollectiveExecution(runtime=runtime, scheduler=scheduler, queue_name=op,
                                   slot_count=slots, credit_window=min(slots, 2),
                                   tile_rows=tile_rows,
                                   workspace_owners=tuple(f"rank{r}" for r in range(world_size)))
