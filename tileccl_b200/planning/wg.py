"""Split of the machine between compute and communication roles, and the task
geometry per TileGroup.  Fields as in the reference (tileccl_v2/wg.py:10-90).  In
the reference a "WG" is a whole SM running one role; the B200 fused kernel keeps
all SMs on the GEMM and gives the communication role to the four epilogue warps
of every CTA, which ``comm_warps_per_cta`` records (``num_comm_wgs = 0`` is then
a valid plan).
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional


@dataclass(frozen=True)
class WGPlan:
    total_sms: int
    num_comm_wgs: int
    max_group_elems: int
    copy_elems: int
    reduce_elems: Optional[int] = None
    packed_values_per_word: int = 4
    comm_warps_per_cta: int = 0

    @property
    def num_comp_wgs(self) -> int:
        return self.total_sms - self.num_comm_wgs

    @property
    def total_wgs(self) -> int:
        return self.total_sms

    @property
    def grid(self) -> tuple:
        return (self.total_wgs,)

    @property
    def copy_qwords(self) -> int:
        return self.copy_elems // self.packed_values_per_word

    @property
    def copy_tasks_per_group(self) -> int:
        return math.ceil(self.max_group_elems / self.copy_elems)

    @property
    def reduce_tasks_per_group(self) -> int:
        return 0 if self.reduce_elems is None else math.ceil(self.max_group_elems / self.reduce_elems)

    @property
    def tasks_per_group(self) -> int:
        return max(self.copy_tasks_per_group, self.reduce_tasks_per_group)

    def to_dict(self) -> dict:
        return {"total_sms": self.total_sms, "num_comm_wgs": self.num_comm_wgs,
                "num_comp_wgs": self.num_comp_wgs, "max_group_elems": self.max_group_elems,
                "copy_elems": self.copy_elems, "reduce_elems": self.reduce_elems,
                "copy_tasks_per_group": self.copy_tasks_per_group,
                "reduce_tasks_per_group": self.reduce_tasks_per_group,
                "comm_warps_per_cta": self.comm_warps_per_cta}


def build_wg_plan(*, total_sms: int, num_comm_wgs: int, max_group_elems: int, copy_elems: int,
                  reduce_elems: Optional[int] = None, packed_values_per_word: int = 4,
                  comm_warps_per_cta: int = 0) -> WGPlan:
    if total_sms <= 0:
        raise ValueError("total_sms must be positive")
    if num_comm_wgs < 0:
        raise ValueError("num_comm_wgs must be non-negative")
    if total_sms - num_comm_wgs <= 0:
        raise ValueError(f"num_comm_wgs={num_comm_wgs} leaves no compute WGs")
    if max_group_elems <= 0:
        raise ValueError("max_group_elems must be positive")
    if copy_elems <= 0:
        raise ValueError("copy_elems must be positive")
    if packed_values_per_word <= 0:
        raise ValueError("packed_values_per_word must be positive")
    if copy_elems % packed_values_per_word:
        raise ValueError("copy_elems must be divisible by packed_values_per_word")
    if max_group_elems % packed_values_per_word:
        raise ValueError("max_group_elems must be divisible by packed_values_per_word")
    if reduce_elems is not None and reduce_elems <= 0:
        raise ValueError("reduce_elems must be positive")
    if comm_warps_per_cta < 0:
        raise ValueError("comm_warps_per_cta must be non-negative")
    return WGPlan(total_sms, num_comm_wgs, max_group_elems, copy_elems, reduce_elems,
                  packed_values_per_word, comm_warps_per_cta)
