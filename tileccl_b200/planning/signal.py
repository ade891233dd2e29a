"""Signal, barrier and trace tensors of one TileGroup-signalled operator.

Counters live on the symmetric heap (peers add to them); trace tensors are
ordinary device tensors that kernels stamp with ``%globaltimer`` values.  Field
names follow the reference (tileccl_v2/signal.py:14-66).  Counters in this
library only grow (targets are multiplied by the call's epoch), so ``reset()`` is
needed only when an operator's epoch is reset too.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Iterable

import torch


@dataclass
class TileGroupSignalState:
    counter: torch.Tensor
    barrier: torch.Tensor
    trace_comm_counter: torch.Tensor
    trace_start_clock: torch.Tensor
    trace_ready_clock: torch.Tensor
    trace_done_clock: torch.Tensor
    extra_counters: dict = field(default_factory=dict)
    epoch: int = 0

    def extra(self, name: str) -> torch.Tensor:
        try:
            return self.extra_counters[name]
        except KeyError:
            raise KeyError(f"unknown TileGroup signal counter: {name}") from None

    def next_epoch(self) -> int:
        self.epoch += 1
        return self.epoch

    def reset(self) -> None:
        self.epoch = 0
        for t in (self.counter, self.barrier, self.trace_comm_counter, self.trace_start_clock,
                  self.trace_ready_clock, self.trace_done_clock, *self.extra_counters.values()):
            t.zero_()


def allocate_tile_group_signals(*, heap, n_groups: int, device, extra_counters: Iterable[str] = ()
                                ) -> TileGroupSignalState:
    if n_groups <= 0:
        raise ValueError("n_groups must be positive")
    extra = {name: heap.allocate_tensor((n_groups,), torch.int32) for name in extra_counters}
    state = TileGroupSignalState(
        counter=heap.allocate_tensor((n_groups,), torch.int32),
        barrier=heap.allocate_tensor((n_groups,), torch.int32),
        trace_comm_counter=torch.zeros((n_groups,), dtype=torch.int32, device=device),
        trace_start_clock=torch.zeros((1,), dtype=torch.int64, device=device),
        trace_ready_clock=torch.zeros((n_groups,), dtype=torch.int64, device=device),
        trace_done_clock=torch.zeros((n_groups,), dtype=torch.int64, device=device),
        extra_counters=extra)
    state.counter.zero_()
    state.barrier.zero_()
    for t in extra.values():
        t.zero_()
    return state
