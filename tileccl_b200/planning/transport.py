"""How a TileGroup travels between ranks: direction (push / pull) and the
granularity of the copy and reduce tasks it is cut into.  API of the reference's
transport plan (tileccl_v2/transport.py:15-86) plus two B200 knobs:
``vector_bytes`` (16-byte accesses) and ``use_multimem`` (NVLS).
"""

from __future__ import annotations

from dataclasses import dataclass
from enum import Enum
from typing import Optional, Union

from .wg import WGPlan, build_wg_plan

PACKED_FP16_VALUES_PER_WORD = 4  # four fp16 values per 64-bit word


class CommMode(Enum):
    PUSH = "push"
    PULL = "pull"


@dataclass(frozen=True)
class P2PTransportPlan:
    comm_mode: CommMode
    copy_elems: int
    reduce_elems: Optional[int] = None
    packed_values_per_word: int = PACKED_FP16_VALUES_PER_WORD
    vector_bytes: int = 16
    use_multimem: bool = False

    @property
    def push_mode(self) -> bool:
        return self.comm_mode is CommMode.PUSH

    @property
    def copy_qwords(self) -> int:
        return self.copy_elems // self.packed_values_per_word

    def build_wg_plan(self, *, total_sms: int, num_comm_wgs: int, max_group_elems: int) -> WGPlan:
        return build_wg_plan(total_sms=total_sms, num_comm_wgs=num_comm_wgs,
                             max_group_elems=max_group_elems, copy_elems=self.copy_elems,
                             reduce_elems=self.reduce_elems,
                             packed_values_per_word=self.packed_values_per_word)

    def to_dict(self) -> dict:
        return {"comm_mode": self.comm_mode.value, "copy_elems": self.copy_elems,
                "reduce_elems": self.reduce_elems,
                "packed_values_per_word": self.packed_values_per_word,
                "vector_bytes": self.vector_bytes, "use_multimem": self.use_multimem}


def normalize_comm_mode(comm_mode: Union[str, CommMode]) -> CommMode:
    if isinstance(comm_mode, CommMode):
        return comm_mode
    for mode in CommMode:
        if mode.value == comm_mode:
            return mode
    allowed = ", ".join(m.value for m in CommMode)
    raise ValueError(f"unknown comm_mode={comm_mode!r}; expected one of {allowed}")


def build_p2p_transport_plan(*, comm_mode: Union[str, CommMode], copy_elems: int,
                             reduce_elems: Optional[int] = None,
                             packed_values_per_word: int = PACKED_FP16_VALUES_PER_WORD,
                             vector_bytes: int = 16, use_multimem: bool = False) -> P2PTransportPlan:
    if copy_elems <= 0:
        raise ValueError("copy_elems must be positive")
    if reduce_elems is not None and reduce_elems <= 0:
        raise ValueError("reduce_elems must be positive")
    if packed_values_per_word <= 0:
        raise ValueError("packed_values_per_word must be positive")
    if vector_bytes not in (4, 8, 16):
        raise ValueError("vector_bytes must be 4, 8 or 16")
    return P2PTransportPlan(normalize_comm_mode(comm_mode), copy_elems, reduce_elems,
                            packed_values_per_word, vector_bytes, use_multimem)
