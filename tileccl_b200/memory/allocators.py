"""Allocation bookkeeping for the symmetric heap.

The bump pointer itself lives in C++ (``csrc/runtime/symm_heap.cc``); this
module holds the Python-visible records and descriptors that the heap reports
through ``metadata()``.  The reference keeps equivalent dataclasses beside its
``TorchBumpAllocator`` (tileccl/memory/allocators.py:30-196, 477-607); the
B200 heap has one segment per rank, backed by one cuMem allocation, exported as
a POSIX file descriptor.
"""

from __future__ import annotations

from dataclasses import asdict, dataclass, field
from typing import Optional

import torch

ALIGNMENT = 256
ALLOCATOR_NAME = "vmm_bump"


def round_up(value: int, alignment: int = ALIGNMENT) -> int:
    return (value + alignment - 1) // alignment * alignment


@dataclass
class AllocationRecord:
    """One tensor carved out of the heap."""

    offset: int
    nbytes: int
    shape: tuple
    dtype: torch.dtype

    def to_dict(self) -> dict:
        return {"offset": self.offset, "nbytes": self.nbytes, "shape": list(self.shape),
                "dtype": str(self.dtype)}


@dataclass(frozen=True)
class MemorySegmentDescriptor:
    """A contiguous device-memory range owned by the allocator."""

    segment_id: str
    segment_kind: str
    allocator_name: str
    base_ptr: int
    size_bytes: int
    device: str

    def to_dict(self) -> dict:
        return asdict(self)


@dataclass(frozen=True)
class AllocatorMemoryModelDescriptor:
    allocator_name: str = ALLOCATOR_NAME
    local_segment_layout: str = "single_vmm_allocation"
    peer_import_model: str = "cuMemImportFromShareableHandle"
    peer_mapping_model: str = "contiguous_window_rank_major"
    external_tensor_import_mode: str = "copy"
    external_mapping_mode: str = "none"

    def to_dict(self) -> dict:
        return asdict(self)


@dataclass(frozen=True)
class AllocatorSegmentLayoutDescriptor:
    allocator_name: str = ALLOCATOR_NAME
    layout_kind: str = "single_segment"
    segment_count: int = 1
    exportable_segment_count: int = 1
    primary_segment_id: str = "heap"
    exportable_segment_ids: tuple = ("heap",)
    multi_segment: bool = False

    def to_dict(self) -> dict:
        d = asdict(self)
        d["exportable_segment_ids"] = list(self.exportable_segment_ids)
        return d


@dataclass(frozen=True)
class ExternalMemoryInterfaceDescriptor:
    allocator_name: str = ALLOCATOR_NAME
    import_mode: str = "copy"
    mapping_mode: str = "none"
    copy_import_supported: bool = True
    zero_copy_mapping_supported: bool = False
    fd_passing: bool = True
    dmabuf_mapping: bool = False

    def to_dict(self) -> dict:
        return asdict(self)


@dataclass(frozen=True)
class PeerMemoryExportDescriptor:
    """What a rank offers to its peers: its heap segment and how it travels."""

    peer_rank: int
    segment_id: str
    segment_kind: str
    allocator_name: str
    transport: str
    size_bytes: int
    base_ptr: int
    device: str
    payload: object = None

    def to_dict(self) -> dict:
        d = asdict(self)
        d.pop("payload")
        d["payload_type"] = type(self.payload).__name__
        return d


@dataclass(frozen=True)
class ImportedPeerMemory:
    """A peer's segment as mapped into this process."""

    peer_rank: int
    segment_id: str
    segment_kind: str
    allocator_name: str
    transport: str
    access_kind: str
    mapped_ptr: int
    exported_base_ptr: int
    size_bytes: int
    device: str
    cleanup_kind: str
    cleanup_resource: Optional[object] = None

    def to_dict(self) -> dict:
        d = asdict(self)
        d.pop("cleanup_resource")
        return d


@dataclass
class BumpLedger:
    """Python mirror of the native bump pointer: keeps per-tensor records and
    lets a debug run compare allocation order across ranks."""

    capacity: int
    records: list = field(default_factory=list)

    def note(self, offset: int, nbytes: int, shape: tuple, dtype: torch.dtype) -> AllocationRecord:
        rec = AllocationRecord(offset, nbytes, tuple(shape), dtype)
        self.records.append(rec)
        return rec

    def reset(self) -> None:
        self.records.clear()

    def fingerprint(self) -> tuple:
        """Order-sensitive digest; equal on every rank iff allocations were symmetric."""
        return tuple((r.offset, r.nbytes) for r in self.records)


class BaseSymmetricAllocator:
    """Interface of a symmetric allocator (capability flags + descriptors)."""

    name = "base"
    supports_external_mapping = False
    supports_fd_passing = False
    supports_dmabuf_mapping = False

    def memory_model(self) -> AllocatorMemoryModelDescriptor:  # pragma: no cover - interface
        raise NotImplementedError

    def capabilities(self) -> dict:
        return {
            "external_mapping": self.supports_external_mapping,
            "fd_passing": self.supports_fd_passing,
            "dmabuf_mapping": self.supports_dmabuf_mapping,
        }


class VmmBumpAllocator(BaseSymmetricAllocator):
    """Descriptor-side view of the native allocator."""

    name = ALLOCATOR_NAME
    supports_fd_passing = True

    def memory_model(self) -> AllocatorMemoryModelDescriptor:
        return AllocatorMemoryModelDescriptor()

    def segment_layout(self) -> AllocatorSegmentLayoutDescriptor:
        return AllocatorSegmentLayoutDescriptor()

    def external_memory_interface(self) -> ExternalMemoryInterfaceDescriptor:
        return ExternalMemoryInterfaceDescriptor()


def create_allocator(allocator_type: str = ALLOCATOR_NAME) -> VmmBumpAllocator:
    """Accepts the reference's names (``torch`` / ``torch_bump``) for API parity."""
    if allocator_type not in (ALLOCATOR_NAME, "torch", "torch_bump", "vmm"):
        raise ValueError(
            f"unknown allocator_type {allocator_type!r}; this build has one allocator: {ALLOCATOR_NAME!r}"
        )
    return VmmBumpAllocator()
