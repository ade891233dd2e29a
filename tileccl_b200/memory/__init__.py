"""Memory substrate: symmetric heap, allocator descriptors, pointer translation."""

from .allocators import (
    ALIGNMENT,
    AllocationRecord,
    AllocatorMemoryModelDescriptor,
    AllocatorSegmentLayoutDescriptor,
    BaseSymmetricAllocator,
    ExternalMemoryInterfaceDescriptor,
    ImportedPeerMemory,
    MemorySegmentDescriptor,
    PeerMemoryExportDescriptor,
    VmmBumpAllocator,
    create_allocator,
)
from .symmetric_heap import PeerMemoryMapEntry, SymmetricHeap
from .translation import PointerTranslator

__all__ = [
    "ALIGNMENT", "AllocationRecord", "AllocatorMemoryModelDescriptor",
    "AllocatorSegmentLayoutDescriptor", "BaseSymmetricAllocator",
    "ExternalMemoryInterfaceDescriptor", "ImportedPeerMemory", "MemorySegmentDescriptor",
    "PeerMemoryExportDescriptor", "VmmBumpAllocator", "create_allocator", "PeerMemoryMapEntry",
    "SymmetricHeap", "PointerTranslator",
]
