"""TileGroup planning layer: collective specs, the TileGroup planner, transport
and role plans, signal state, the alpha-beta cost model and the timeline recorder.

Importable as ``tileccl_v2`` for code written against the reference's package of
that name (tileccl_v2/__init__.py:61-103); nothing here needs a GPU.
"""

from .collective_spec import CollectiveKind, CollectiveSpec, all_gather_spec, reduce_scatter_spec
from .cost_model import (CalibrationPoint, CostModelCalibrator, HardwareProfile, Interconnect,
                         PipelineCost, TileCost, TileCostModel)
from .heap import SymmetricHeap
from .runtime.timeline import TimelineEvent, TimelineRecorder
from .signal import TileGroupSignalState, allocate_tile_group_signals
from .tile_group import (DEFAULT_BLOCK_M, DEFAULT_BLOCK_N, DEFAULT_GROUP_M, DEFAULT_TAU_MIN_BYTES,
                         TileGroup, TileGroupPlan, build_group_table, build_tile_group_plan,
                         build_tile_groups, plan_for_fused_kernel, split_groups_at_row_boundaries,
                         split_groups_at_row_shards)
from .transport import CommMode, P2PTransportPlan, build_p2p_transport_plan, normalize_comm_mode
from .wg import WGPlan, build_wg_plan

__version__ = "2.3.0-b200"

__all__ = [
    "CollectiveKind", "CollectiveSpec", "all_gather_spec", "reduce_scatter_spec",
    "CalibrationPoint", "CostModelCalibrator", "HardwareProfile", "Interconnect", "PipelineCost",
    "TileCost", "TileCostModel", "SymmetricHeap", "TimelineEvent", "TimelineRecorder",
    "TileGroupSignalState", "allocate_tile_group_signals", "DEFAULT_BLOCK_M", "DEFAULT_BLOCK_N",
    "DEFAULT_GROUP_M", "DEFAULT_TAU_MIN_BYTES", "TileGroup", "TileGroupPlan", "build_group_table",
    "build_tile_group_plan", "build_tile_groups", "plan_for_fused_kernel",
    "split_groups_at_row_boundaries", "split_groups_at_row_shards", "CommMode", "P2PTransportPlan",
    "build_p2p_transport_plan", "normalize_comm_mode", "WGPlan", "build_wg_plan",
]
