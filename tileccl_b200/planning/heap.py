"""The planning package's heap is the library's one symmetric heap.

The reference ships a second, slimmer heap class in its v2 package
(tileccl_v2/heap.py:88-388); its extra methods (``allocate_signal_buffer``,
``reset_allocator``, ``bytes_used``, ``local_ptr``) exist on
:class:`tileccl_b200.memory.SymmetricHeap`, so one class serves both APIs.
"""

from ..memory.symmetric_heap import SymmetricHeap

__all__ = ["SymmetricHeap"]
