"""Host-side pointer translation between ranks' heaps.

On the device, translation is ``ptr + (to - from) * stride`` (see
``csrc/device/symm_ptr.cuh``); this class does the same arithmetic on the host
with bounds checking, for launchers and tests.  It keeps the method names of
the reference's ``PointerTranslator`` (tileccl/memory/translation.py:296-452).
"""

from __future__ import annotations

from typing import Sequence


class PointerTranslator:
    def __init__(self, heap_bases: Sequence[int], heap_size: int):
        bases = [int(b) for b in heap_bases]
        if not bases:
            raise ValueError("heap_bases must not be empty")
        if heap_size <= 0:
            raise ValueError("heap_size must be positive")
        self._bases = bases
        self._size = int(heap_size)

    @classmethod
    def from_heap(cls, heap) -> "PointerTranslator":
        return cls([heap.peer_base(r) for r in range(heap.world_size)], heap.size)

    @property
    def world_size(self) -> int:
        return len(self._bases)

    def base(self, rank: int) -> int:
        self._check_rank(rank)
        return self._bases[rank]

    def get_offset(self, ptr: int, rank: int) -> int:
        """Offset of ``ptr`` inside ``rank``'s heap; ``ValueError`` if outside."""
        self._check_rank(rank)
        off = int(ptr) - self._bases[rank]
        if off < 0 or off >= self._size:
            raise ValueError(
                f"pointer 0x{int(ptr):x} is not inside rank {rank}'s heap "
                f"(base 0x{self._bases[rank]:x}, size {self._size})")
        return off

    def validate(self, ptr: int, rank: int, nbytes: int = 1) -> bool:
        self._check_rank(rank)
        off = int(ptr) - self._bases[rank]
        return 0 <= off and off + max(int(nbytes), 1) <= self._size

    def translate(self, ptr: int, from_rank: int, to_rank: int) -> int:
        off = self.get_offset(ptr, from_rank)
        self._check_rank(to_rank)
        return self._bases[to_rank] + off

    def _check_rank(self, rank: int) -> None:
        if rank < 0 or rank >= len(self._bases):
            raise ValueError(f"rank {rank} out of range for world_size {len(self._bases)}")
