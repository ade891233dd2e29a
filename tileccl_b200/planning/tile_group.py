"""TileGroup planning API (the policy itself is C++: ``csrc/plan/tile_group.cc``).

Signatures and defaults follow the reference planner
(tileccl_v2/tile_group.py:19-301): ``build_tile_groups``,
``split_groups_at_row_boundaries``, ``split_groups_at_row_shards``,
``build_group_table``, ``build_tile_group_plan`` and ``TileGroupPlan``.
``plan_for_fused_kernel`` adds what the B200 kernel needs: its tile is
128 x 256, and its TileGroups are uniform bands of ``group_m_tiles`` tile rows.
"""

from __future__ import annotations

import ctypes as C
import math
from dataclasses import dataclass
from typing import Optional, Sequence

import torch

from .. import _native

DEFAULT_BLOCK_M = 128
DEFAULT_BLOCK_N = 128
DEFAULT_GROUP_M = 8
DEFAULT_TAU_MIN_BYTES = 262144

TileGroup = tuple  # (row_start, row_end, tile_count)


@dataclass(frozen=True)
class TileGroupPlan:
    M: int
    N: int
    tile_bytes: int
    target_group_tiles: Optional[int]
    max_groups: int
    groups: list
    group_table: torch.Tensor
    block_m: int = DEFAULT_BLOCK_M
    block_n: int = DEFAULT_BLOCK_N
    group_m: int = DEFAULT_GROUP_M
    tau_min_bytes: int = DEFAULT_TAU_MIN_BYTES
    p0_min_tiles: int = 1

    @property
    def n_groups(self) -> int:
        return len(self.groups)

    @property
    def max_rb(self) -> int:
        """Most tile rows in any group."""
        return max(math.ceil((e - s) / self.block_m) for s, e, _ in self.groups)

    @property
    def max_cb(self) -> int:
        """Tile columns."""
        return math.ceil(self.N / self.block_n)

    @property
    def max_group_elems(self) -> int:
        return max((e - s) * self.N for s, e, _ in self.groups)

    @property
    def min_group_tiles(self) -> int:
        return min(t for _, _, t in self.groups)

    @property
    def max_group_tiles(self) -> int:
        return max(t for _, _, t in self.groups)

    @property
    def avg_group_tiles(self) -> float:
        return sum(t for _, _, t in self.groups) / len(self.groups)

    def row_starts(self) -> list:
        return [s for s, _, _ in self.groups]

    def row_ends(self) -> list:
        return [min(e, self.M) for _, e, _ in self.groups]

    def tile_counts(self) -> list:
        return [t for _, _, t in self.groups]

    def to_dict(self) -> dict:
        return {"M": self.M, "N": self.N, "tile_bytes": self.tile_bytes, "n_groups": self.n_groups,
                "groups": [list(g) for g in self.groups], "block_m": self.block_m,
                "block_n": self.block_n, "group_m": self.group_m,
                "tau_min_bytes": self.tau_min_bytes, "p0_min_tiles": self.p0_min_tiles}


def _native_groups(M, N, tile_bytes, target_group_tiles, max_groups, block_m, block_n, group_m,
                   tau_min_bytes, boundaries) -> list:
    for name, v in (("M", M), ("N", N)):
        if v <= 0:
            raise ValueError("M and N must be positive")
    if tile_bytes <= 0:
        raise ValueError("tile_bytes must be positive")
    if block_m <= 0 or block_n <= 0 or group_m <= 0:
        raise ValueError("block_m, block_n, and group_m must be positive")
    if max_groups <= 0:
        raise ValueError("max_groups must be positive")
    bounds = [int(b) for b in boundaries]
    cap = math.ceil(M / block_m) + len(bounds) + 2
    out = (C.c_int64 * (3 * cap))()
    n = C.c_int32()
    barr = (C.c_int64 * max(1, len(bounds)))(*bounds) if bounds else None
    _native.call("tccl_plan_tile_groups", int(M), int(N), int(tile_bytes),
                 int(target_group_tiles or 0), int(max_groups), int(block_m), int(block_n),
                 int(group_m), int(tau_min_bytes), barr, len(bounds), out, cap, C.byref(n))
    return [(out[3 * i], out[3 * i + 1], out[3 * i + 2]) for i in range(n.value)]


def build_tile_groups(M: int, N: int, tile_bytes: int, *, target_group_tiles: Optional[int] = None,
                      max_groups: int = 64, block_m: int = DEFAULT_BLOCK_M,
                      block_n: int = DEFAULT_BLOCK_N, group_m: int = DEFAULT_GROUP_M,
                      tau_min_bytes: int = DEFAULT_TAU_MIN_BYTES) -> list:
    """Wave-aligned row bands of at least ``ceil(tau_min_bytes / tile_bytes)`` tiles each."""
    return _native_groups(M, N, tile_bytes, target_group_tiles, max_groups, block_m, block_n,
                          group_m, tau_min_bytes, ())


def split_groups_at_row_boundaries(M: int, N: int, groups: Sequence[tuple],
                                   row_boundaries: Sequence[int], *,
                                   block_m: int = DEFAULT_BLOCK_M,
                                   block_n: int = DEFAULT_BLOCK_N) -> list:
    """Cut groups so that none contains a boundary row in its interior."""
    tile_cols = math.ceil(N / block_n)
    cuts = sorted({M, *(b for b in row_boundaries if 0 < b < M)})
    out = []
    for start, raw_end, _ in groups:
        end = min(raw_end, M)
        at = start
        while at < end:
            stop = min(end, next(c for c in cuts if c > at))
            out.append((at, stop, math.ceil((stop - at) / block_m) * tile_cols))
            at = stop
    return out


def split_groups_at_row_shards(M: int, N: int, groups: Sequence[tuple], *, num_shards: int,
                               block_m: int = DEFAULT_BLOCK_M,
                               block_n: int = DEFAULT_BLOCK_N) -> list:
    if num_shards <= 0:
        raise ValueError("num_shards must be positive")
    if M % num_shards:
        raise ValueError(f"M={M} must be divisible by num_shards={num_shards}")
    per = M // num_shards
    return split_groups_at_row_boundaries(M, N, groups, [per * s for s in range(1, num_shards)],
                                          block_m=block_m, block_n=block_n)


def build_group_table(M: int, N: int, groups: Sequence[tuple], *, block_m: int = DEFAULT_BLOCK_M,
                      block_n: int = DEFAULT_BLOCK_N, group_m: int = DEFAULT_GROUP_M) -> torch.Tensor:
    """int32[tiles]: tile id (group_m-swizzled rasterisation) -> TileGroup id."""
    tiles = math.ceil(M / block_m) * math.ceil(N / block_n)
    flat = (C.c_int64 * max(1, 3 * len(groups)))(*[int(x) for g in groups for x in g])
    table = torch.zeros(tiles, dtype=torch.int32)
    ptr = C.cast(table.data_ptr(), C.POINTER(C.c_int32))
    _native.call("tccl_plan_group_table", int(M), int(N), flat, len(groups), int(block_m),
                 int(block_n), int(group_m), ptr, tiles)
    return table


def build_tile_group_plan(M: int, N: int, tile_bytes: int, *,
                          target_group_tiles: Optional[int] = None, max_groups: int = 64,
                          block_m: int = DEFAULT_BLOCK_M, block_n: int = DEFAULT_BLOCK_N,
                          group_m: int = DEFAULT_GROUP_M, tau_min_bytes: int = DEFAULT_TAU_MIN_BYTES,
                          row_split_boundaries: Sequence[int] = ()) -> TileGroupPlan:
    groups = _native_groups(M, N, tile_bytes, target_group_tiles, max_groups, block_m, block_n,
                            group_m, tau_min_bytes, tuple(row_split_boundaries))
    table = build_group_table(M, N, groups, block_m=block_m, block_n=block_n, group_m=group_m)
    return TileGroupPlan(M=M, N=N, tile_bytes=tile_bytes, target_group_tiles=target_group_tiles,
                         max_groups=max_groups, groups=groups, group_table=table, block_m=block_m,
                         block_n=block_n, group_m=group_m, tau_min_bytes=tau_min_bytes,
                         p0_min_tiles=max(1, math.ceil(tau_min_bytes / tile_bytes)))


def plan_for_fused_kernel(rows: int, cols: int, *, elem_bytes: int = 2,
                          tau_min_bytes: int = DEFAULT_TAU_MIN_BYTES, max_groups: int = 64) -> dict:
    """TileGroup geometry for the sm_100a fused kernel (128 x 256 tiles, uniform bands).

    Returns ``group_m_tiles`` (tile rows per group, what the kernel takes) together
    with the plan it was derived from.
    """
    bm, bn = 128, 256
    tile_bytes = bm * bn * elem_bytes
    tile_cols = math.ceil(cols / bn)
    need_rows = max(1, math.ceil(math.ceil(tau_min_bytes / tile_bytes) / tile_cols))
    tile_rows = math.ceil(rows / bm)
    group_m_tiles = max(need_rows, math.ceil(tile_rows / max_groups))
    plan = build_tile_group_plan(rows, cols, tile_bytes, block_m=bm, block_n=bn,
                                 group_m=group_m_tiles, tau_min_bytes=tau_min_bytes,
                                 max_groups=max_groups)
    return {"group_m_tiles": group_m_tiles, "n_groups": math.ceil(tile_rows / group_m_tiles),
            "plan": plan}
