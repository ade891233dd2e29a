"""Symmetric heap: the same amount of device memory on every rank, every rank's
copy mapped into every process, so device code can address a peer's copy of any
heap object.

Python face of ``csrc/runtime/symm_heap.cc``.  API follows the reference heap
(tileccl/memory/symmetric_heap.py:124-1358) so that code written against it
keeps working: ``SymmetricHeap(size, rank, world_size)``,
``SymmetricHeap.create_all``, ``allocate_tensor``, ``get_heap_bases``,
``translate``, ``barrier``, ``cleanup``, ``metadata`` ...  What differs:

* memory comes from cuMem VMM, not ``torch.empty``; peers are mapped from
  file-descriptor handles, not CUDA IPC handles
  (``transport_strategy`` is ``vmm_single_process`` / ``vmm_fd``);
* all ranks sit in one contiguous virtual window, so ``heap_bases[r]`` is
  ``window_base + r * stride`` and kernels translate with arithmetic only;
* ``multicast_base`` is the NVLS alias of the heap when the devices support it;
* ``create_all`` accepts more ranks than there are GPUs: the extra ranks share
  devices ("emulated ranks"), which is how multi-rank logic is exercised on a
  single GPU.
"""

from __future__ import annotations

import ctypes as C
import logging
import os
import uuid
from dataclasses import dataclass, field
from typing import Optional, Sequence

import torch

from .. import _native
from .allocators import (
    ALIGNMENT,
    BumpLedger,
    ImportedPeerMemory,
    MemorySegmentDescriptor,
    PeerMemoryExportDescriptor,
    VmmBumpAllocator,
    create_allocator,
)

logger = logging.getLogger(__name__)

_MODE_NAMES = {0: "local_only", 1: "single_process", 2: "multiprocess"}
_TRANSPORT_NAMES = {0: "local_only", 1: "vmm_single_process", 2: "vmm_fd", 3: "vmm_fabric"}


def _human_bytes(n: int) -> str:
    for unit in ("B", "KiB", "MiB", "GiB"):
        if n < 1024 or unit == "GiB":
            return f"{n:.1f} {unit}" if unit != "B" else f"{n} B"
        n /= 1024
    return f"{n} B"


class _DeviceRange:
    """Exposes a raw device address range through ``__cuda_array_interface__``."""

    def __init__(self, ptr: int, nbytes: int, keepalive: object):
        self._keepalive = keepalive
        self.__cuda_array_interface__ = {
            "shape": (nbytes,),
            "typestr": "|u1",
            "data": (ptr, False),
            "version": 3,
            "strides": None,
        }


@dataclass(frozen=True)
class PeerMemoryMapEntry:
    """Where rank ``peer_rank``'s heap is mapped in this process."""

    peer_rank: int
    mapped_ptr: int
    size_bytes: int
    transport: str
    access_kind: str
    is_local: bool

    def to_dict(self) -> dict:
        return {
            "peer_rank": self.peer_rank,
            "mapped_ptr": self.mapped_ptr,
            "size_bytes": self.size_bytes,
            "transport": self.transport,
            "access_kind": self.access_kind,
            "is_local": self.is_local,
        }


@dataclass
class LocalGroup:
    """The ranks that one process drives (``SymmetricHeap.create_all`` / ``init_local``).

    ``emulated`` is true when some ranks share a GPU.  Kernels of different ranks
    must then never wait on each other inside a launch, so multi-rank operators
    park their per-rank launches in ``pending`` and replay them phase by phase
    once every rank has called.
    """

    world_size: int
    devices: list
    contexts: list = field(default_factory=list)
    pending: dict = field(default_factory=dict)

    @property
    def emulated(self) -> bool:
        return len(set(self.devices)) < len(self.devices)


class _NativeHandle:
    """Owns one native heap handle; destroying the last one unmaps the window."""

    def __init__(self, handle: C.c_void_p):
        self.handle = handle

    def close(self) -> None:
        if self.handle:
            _native.call("tccl_heap_destroy", self.handle)
            self.handle = None

    def __del__(self):  # pragma: no cover - best effort
        try:
            self.close()
        except Exception:
            pass


class SymmetricHeap:
    """One rank's view of the symmetric heap."""

    def __init__(self, size: int, rank: int, world_size: int, backend: str = "auto", *,
                 allocator_type: str = "vmm_bump", device: Optional[int] = None,
                 nvls: Optional[bool] = None, _handle: Optional[C.c_void_p] = None,
                 _group=None) -> None:
        if size <= 0:
            raise ValueError(f"Heap size must be positive, got {size}")
        if world_size < 1:
            raise ValueError(f"world_size must be >= 1, got {world_size}")
        if rank < 0 or rank >= world_size:
            raise ValueError(f"rank={rank} out of range for world_size={world_size}")
        if backend not in ("auto", "cuda"):
            raise ValueError(
                f"backend {backend!r} is not available: this library targets NVIDIA B200 (CUDA) only")
        self._size = int(size)
        self._rank = int(rank)
        self._world_size = int(world_size)
        self._backend_name = "cuda"
        self._allocator: VmmBumpAllocator = create_allocator(allocator_type)
        self._cleaned_up = False
        self._group = _group
        self.local_group: Optional[LocalGroup] = None
        self._state: dict = {}
        self._reset_hooks: list = []
        self._dirty = False  # True once reset_allocator() may have exposed used memory
        want_nvls = _want_nvls(nvls)

        if _handle is None:
            if not torch.cuda.is_available():
                raise RuntimeError("SymmetricHeap needs a CUDA device (torch.cuda.is_available() is False)")
            if world_size == 1:
                dev = torch.cuda.current_device() if device is None else int(device)
                devices = (C.c_int32 * 1)(dev)
                out = (C.c_void_p * 1)()
                _native.call("tccl_heap_create_local", 1, self._size, devices, 0, out)
                _handle = C.c_void_p(out[0])
            else:
                _handle = self._create_multiprocess(device, want_nvls)
        self._native = _NativeHandle(_handle)

        info = _native.HeapInfo()
        _native.call("tccl_heap_info", self._native.handle, C.byref(info))
        self._info = info
        self._device = torch.device("cuda", info.device)
        self._window_base = int(info.window_base)
        self._stride = int(info.stride)
        self._mc_base = int(info.mc_base)
        self._mode = _MODE_NAMES.get(info.mode, "unknown")
        self._transport_strategy = _TRANSPORT_NAMES.get(info.transport, "unknown")
        self._local_ptr = self._window_base + self._rank * self._stride
        self._ledger = BumpLedger(capacity=self._size)
        self._buffer = torch.as_tensor(_DeviceRange(self._local_ptr, self._size, self._native),
                                       device=self._device)
        self._peer_buffers: dict[int, torch.Tensor] = {self._rank: self._buffer}
        self._heap_bases: Optional[torch.Tensor] = None
        logger.info("rank %d: symmetric heap %s on %s (%s, %s, nvls=%s)", self._rank,
                    _human_bytes(self._size), self._device, self._mode, self._transport_strategy,
                    bool(self._mc_base))

    # ------------------------------------------------------------ construction
    def _create_multiprocess(self, device: Optional[int], want_nvls: bool) -> C.c_void_p:
        import torch.distributed as dist

        if not dist.is_initialized():
            raise RuntimeError(
                "multi-process SymmetricHeap needs torch.distributed to be initialised "
                "(it is only used to agree on a rendezvous name)")
        dev = torch.cuda.current_device() if device is None else int(device)
        # Rank 0 picks the rendezvous name; everybody learns it.
        box = [f"{os.getpid()}-{uuid.uuid4().hex[:12]}" if self._rank == 0 else None]
        dist.broadcast_object_list(box, src=0, group=self._group)
        job_id = str(box[0])
        from ..utils.config import current

        timeout_ms = current().bootstrap_timeout_ms or 120000
        out = C.c_void_p()
        _native.call("tccl_heap_create_multiprocess", self._rank, self._world_size, self._size, dev,
                     job_id.encode(), 1 if want_nvls else 0, timeout_ms, C.byref(out))
        return out

    @classmethod
    def create_all(cls, size: int, world_size: int, backend: str = "auto", *,
                   allocator_type: str = "vmm_bump", devices: Optional[Sequence[int]] = None,
                   nvls: Optional[bool] = None) -> list["SymmetricHeap"]:
        """Single-process mode: one heap per rank, all mapped in this process.

        Rank ``r`` lives on ``devices[r]`` (default ``r % device_count``).
        """
        if world_size < 1:
            raise ValueError(f"world_size must be >= 1, got {world_size}")
        if size <= 0:
            raise ValueError(f"Heap size must be positive, got {size}")
        if not torch.cuda.is_available():
            raise RuntimeError("SymmetricHeap.create_all needs at least one CUDA device")
        ndev = torch.cuda.device_count()
        if devices is None:
            devices = [r % ndev for r in range(world_size)]
        if len(devices) != world_size:
            raise ValueError("devices must have one entry per rank")
        arr = (C.c_int32 * world_size)(*[int(d) for d in devices])
        out = (C.c_void_p * world_size)()
        _native.call("tccl_heap_create_local", world_size, int(size), arr,
                     1 if _want_nvls(nvls) else 0, out)
        heaps = [cls(size, r, world_size, backend, allocator_type=allocator_type,
                     _handle=C.c_void_p(out[r])) for r in range(world_size)]
        group = LocalGroup(world_size=world_size, devices=[int(d) for d in devices])
        for h in heaps:
            h.local_group = group
        return heaps

    # -------------------------------------------------------------- allocation
    def allocate_tensor(self, shape, dtype: torch.dtype) -> torch.Tensor:
        """Carve a tensor out of the heap (256-byte aligned, never freed).

        Collective by contract: every rank must allocate the same shapes in the
        same order so that equal offsets name the same object everywhere.
        """
        self._check_alive()
        if isinstance(shape, int):
            shape = (shape,)
        shape = tuple(int(s) for s in shape)
        numel = 1
        for s in shape:
            if s < 0:
                raise ValueError(f"negative dimension in shape {shape}")
            numel *= s
        itemsize = torch.empty((), dtype=dtype).element_size()
        nbytes = numel * itemsize
        off = C.c_uint64()
        _native.call("tccl_heap_alloc", self._native.handle, nbytes, C.byref(off))
        offset = int(off.value)
        self._ledger.note(offset, nbytes, shape, dtype)
        flat = self._buffer[offset:offset + nbytes]
        return flat.view(dtype).view(shape)

    def allocate_zeroed(self, shape, dtype: torch.dtype) -> torch.Tensor:
        """A tensor that is zero on every rank before any peer can write to it.

        The heap is zeroed when it is created, before peers can reach it, and bump
        allocations are never reused, so fresh memory is already zero and no memset
        is issued: a memset by the owner could run after a faster peer has stored a
        signal or data here and wipe it.  Only after ``reset_allocator`` may memory
        be dirty; then every rank zeroes and the ranks meet in a barrier.
        """
        t = self.allocate_tensor(shape, dtype)
        if self._dirty:
            t.zero_()
            self.barrier()
        return t

    def allocate_signal_buffer(self, n: int) -> torch.Tensor:
        """Zeroed int32 flags / counters on the heap (see ``allocate_zeroed``)."""
        return self.allocate_zeroed((int(n),), torch.int32)

    def reset_allocator(self) -> None:
        """Rewind the bump pointer.  Tensors handed out earlier become aliases; every
        rank must have finished using them (call ``barrier()`` first).

        Collective: every rank resets at the same point of its program.  Everything the
        library itself carved from the heap goes with the user tensors: the collectives'
        counter blocks, staging areas and epochs kept here, and (through the reset hooks
        that contexts register) the fused operators' signal blocks, staging, native plans
        and workspaces.  They are re-created, zeroed, on next use, so a tensor allocated
        after the reset can never alias a live counter.
        """
        self._check_alive()
        used = self.bytes_allocated
        _native.call("tccl_heap_reset", self._native.handle)
        self._ledger.reset()
        # Everything handed out so far goes back to zero right here, while no rank is using
        # the heap, so that counters carved from it later need no memset of their own (a late
        # memset by the owner could wipe a signal that a faster peer has already sent).
        if used:
            self._buffer[:used].zero_()
        self._dirty = False
        self.barrier()
        self._state.clear()
        for ref in list(self._reset_hooks):
            hook = ref()
            if hook is None:
                self._reset_hooks.remove(ref)
            else:
                hook()

    def register_reset_hook(self, bound_method) -> None:
        """Call ``bound_method()`` whenever ``reset_allocator`` runs (held weakly)."""
        import weakref

        self._reset_hooks.append(weakref.WeakMethod(bound_method))

    # ---------------------------------------------------------------- queries
    def get_heap_bases(self) -> torch.Tensor:
        """int64[world_size] device tensor: address of each rank's heap in this process."""
        self._check_alive()
        if self._heap_bases is None:
            bases = [self._window_base + r * self._stride for r in range(self._world_size)]
            self._heap_bases = torch.tensor(bases, dtype=torch.int64, device=self._device)
        return self._heap_bases

    heap_bases = property(get_heap_bases)

    @property
    def local_base(self) -> int:
        return self._local_ptr

    local_ptr = local_base

    @property
    def window_base(self) -> int:
        return self._window_base

    @property
    def stride(self) -> int:
        """Bytes between consecutive ranks' heaps in the window."""
        return self._stride

    @property
    def multicast_base(self) -> int:
        """Address of the NVLS alias of the heap, 0 when multicast is not bound."""
        return self._mc_base

    @property
    def has_multicast(self) -> bool:
        return self._mc_base != 0

    @property
    def emulated(self) -> bool:
        """True when this rank shares its GPU with another rank of the same process."""
        return self.local_group is not None and self.local_group.emulated

    @property
    def is_single_process(self) -> bool:
        return self._mode != "multiprocess"

    @property
    def size(self) -> int:
        return self._size

    @property
    def rank(self) -> int:
        return self._rank

    @property
    def world_size(self) -> int:
        return self._world_size

    @property
    def device(self) -> torch.device:
        return self._device

    @property
    def bytes_allocated(self) -> int:
        self._check_alive()
        out = C.c_uint64()
        _native.call("tccl_heap_bytes_allocated", self._native.handle, C.byref(out))
        return int(out.value)

    bytes_used = bytes_allocated

    @property
    def bytes_free(self) -> int:
        return self._size - self.bytes_allocated

    @property
    def mode(self) -> str:
        return self._mode

    @property
    def transport_strategy(self) -> str:
        return self._transport_strategy

    @property
    def allocator_name(self) -> str:
        return self._allocator.name

    def peer_base(self, rank: int) -> int:
        self._validate_rank(rank)
        return self._window_base + rank * self._stride

    def get_peer_buffer(self, rank: int) -> torch.Tensor:
        """uint8 view of ``rank``'s whole heap as mapped here (all modes: the window
        always maps every rank)."""
        self._check_alive()
        self._validate_rank(rank)
        buf = self._peer_buffers.get(rank)
        if buf is None:
            buf = torch.as_tensor(_DeviceRange(self.peer_base(rank), self._size, self._native))
            self._peer_buffers[rank] = buf
        return buf

    def peer_view(self, tensor: torch.Tensor, rank: int) -> torch.Tensor:
        """The tensor that occupies the same heap offset on ``rank``."""
        off = self.get_offset(tensor.data_ptr())
        nbytes = tensor.numel() * tensor.element_size()
        if not tensor.is_contiguous():
            raise ValueError("peer_view needs a contiguous tensor")
        return self.get_peer_buffer(rank)[off:off + nbytes].view(tensor.dtype).view(tensor.shape)

    def owns_tensor(self, tensor: torch.Tensor) -> bool:
        if not tensor.is_cuda:
            return False
        ptr = tensor.data_ptr()
        nbytes = tensor.numel() * tensor.element_size()
        return self._local_ptr <= ptr and ptr + nbytes <= self._local_ptr + self._size

    is_symmetric = owns_tensor

    def import_external_tensor(self, tensor: torch.Tensor) -> torch.Tensor:
        """Copy a tensor into the heap (there is no zero-copy adoption)."""
        out = self.allocate_tensor(tuple(tensor.shape), tensor.dtype)
        out.copy_(tensor)
        return out

    def as_symmetric(self, tensor: torch.Tensor) -> torch.Tensor:
        return tensor if self.owns_tensor(tensor) else self.import_external_tensor(tensor)

    def translate(self, local_ptr: int, to_rank: int) -> int:
        self._validate_rank(to_rank)
        off = self.get_offset(local_ptr)
        return self.peer_base(to_rank) + off

    def get_offset(self, ptr: int) -> int:
        off = int(ptr) - self._local_ptr
        if off < 0 or off >= self._size:
            raise ValueError(
                f"pointer 0x{int(ptr):x} is outside rank {self._rank}'s heap "
                f"[0x{self._local_ptr:x}, 0x{self._local_ptr + self._size:x})")
        return off

    def multicast_ptr(self, local_ptr: int) -> int:
        if not self._mc_base:
            raise RuntimeError("no NVLS multicast mapping is bound to this heap")
        return self._mc_base + self.get_offset(local_ptr)

    # --------------------------------------------------------------- metadata
    def segment_descriptors(self) -> tuple:
        return (MemorySegmentDescriptor("heap", "device_heap", self._allocator.name, self._local_ptr,
                                        self._size, str(self._device)),)

    def peer_export_descriptors(self) -> tuple:
        return tuple(
            PeerMemoryExportDescriptor(r, "heap", "device_heap", self._allocator.name,
                                       self._transport_strategy, self._size, self.peer_base(r),
                                       str(self._device) if r == self._rank else "peer",
                                       payload="posix_fd" if self._mode == "multiprocess" else None)
            for r in range(self._world_size))

    def peer_imports(self) -> tuple:
        return tuple(
            ImportedPeerMemory(r, "heap", "device_heap", self._allocator.name,
                               self._transport_strategy,
                               "local" if r == self._rank else "mapped_remote", self.peer_base(r),
                               self.peer_base(r), self._size,
                               str(self._device) if r == self._rank else "peer",
                               "none" if r == self._rank else "cuMemUnmap")
            for r in range(self._world_size))

    def peer_memory_map(self) -> tuple:
        return tuple(
            PeerMemoryMapEntry(r, self.peer_base(r), self._size, self._transport_strategy,
                               "local" if r == self._rank else "mapped_remote", r == self._rank)
            for r in range(self._world_size))

    def allocator_metadata(self) -> dict:
        return {
            "name": self._allocator.name,
            "alignment": ALIGNMENT,
            "bytes_allocated": self.bytes_allocated if not self._cleaned_up else 0,
            "capacity": self._size,
            "allocations": len(self._ledger.records),
            "capabilities": self._allocator.capabilities(),
        }

    def allocation_fingerprint(self) -> tuple:
        return self._ledger.fingerprint()

    def metadata(self) -> dict:
        """Structured description of the heap for diagnostics and docs."""
        return {
            "rank": self._rank,
            "world_size": self._world_size,
            "backend": self._backend_name,
            "device": str(self._device),
            "size_bytes": self._size,
            "local_base": self._local_ptr,
            "window_base": self._window_base,
            "stride_bytes": self._stride,
            "granularity": int(self._info.granularity),
            "mode": self._mode,
            "transport_strategy": self._transport_strategy,
            "nvls_multicast": bool(self._mc_base),
            "multicast_base": self._mc_base,
            "allocator": self.allocator_metadata(),
            "memory_model": self._allocator.memory_model().to_dict(),
            "external_memory_interface": self._allocator.external_memory_interface().to_dict(),
            "segment_layout": self._allocator.segment_layout().to_dict(),
            "segments": [s.to_dict() for s in self.segment_descriptors()],
            "peer_exports": [p.to_dict() for p in self.peer_export_descriptors()],
            "peer_imports": [p.to_dict() for p in self.peer_imports()],
            "peer_memory_map": [p.to_dict() for p in self.peer_memory_map()],
        }

    # ------------------------------------------------------------- life cycle
    def barrier(self) -> None:
        """All work on this rank's device is done and every rank has arrived."""
        self._check_alive()
        if self._mode == "multiprocess":
            import torch.distributed as dist

            torch.cuda.synchronize(self._device)
            dist.barrier(group=self._group)
        else:
            # One process drives every rank: device-wide synchronisation is the barrier.
            for d in range(torch.cuda.device_count()):
                torch.cuda.synchronize(d)

    def check_symmetric_allocations(self) -> None:
        """Debug aid: raise if ranks allocated different sizes / orders (multi-process)."""
        if self._mode != "multiprocess":
            return
        import torch.distributed as dist

        prints = [None] * self._world_size
        dist.all_gather_object(prints, self.allocation_fingerprint(), group=self._group)
        for r, fp in enumerate(prints):
            if fp != prints[0]:
                raise RuntimeError(
                    f"symmetric heap allocation order differs between rank 0 and rank {r}")

    def cleanup(self) -> None:
        """Unmap and release.  Idempotent.  Tensors from this heap must not be used after."""
        if self._cleaned_up:
            return
        self._cleaned_up = True
        self._heap_bases = None
        self._peer_buffers = {}
        self._buffer = None
        try:
            if torch.cuda.is_available():
                torch.cuda.synchronize(self._device)
        finally:
            self._native.close()

    def _check_alive(self) -> None:
        if self._cleaned_up:
            raise RuntimeError("this SymmetricHeap has been cleaned up")

    def _validate_rank(self, rank: int, label: str = "rank") -> None:
        if rank < 0 or rank >= self._world_size:
            raise ValueError(f"{label}={rank} out of range for world_size={self._world_size}")

    def __enter__(self) -> "SymmetricHeap":
        return self

    def __exit__(self, *exc) -> None:
        self.cleanup()

    def __repr__(self) -> str:
        return (f"SymmetricHeap(rank={self._rank}, world_size={self._world_size}, "
                f"size={_human_bytes(self._size)}, mode={self._mode}, "
                f"transport={self._transport_strategy}, nvls={bool(self._mc_base)})")


def _want_nvls(flag: Optional[bool]) -> bool:
    if flag is not None:
        return bool(flag)
    from ..utils.config import current

    return current().nvls_allowed
