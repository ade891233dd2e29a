"""tileccl_b200 - tile-granular collective communication for NVIDIA B200.

Public entry points (same as the reference's ``tileccl`` package,
tileccl/__init__.py:35-552):

* :func:`init` - one process per GPU (under ``torchrun``) or a single rank;
* :func:`init_local` - one process driving ``world_size`` ranks;
* :class:`TileCCLContext` with the symmetric-heap allocators
  ``ctx.empty / zeros / randn / workspace``;
* ``tileccl_b200.ops`` (fused GEMM + collective operators and collectives),
  ``tileccl_b200.patterns``, ``tileccl_b200.planning`` (TileGroup planner and
  cost model), loaded lazily so that importing the package needs no GPU.

``import tileccl`` / ``import tileccl_v2`` resolve to thin aliases of this
package for code written against the reference.
"""

from __future__ import annotations

import importlib
import os
from dataclasses import dataclass, field
from typing import Any, Optional

__version__ = "0.1.0"

_ctx: Optional["TileCCLContext"] = None

_LAZY_SUBMODULES = ("ops", "patterns", "planning", "primitives", "sync", "memory", "utils",
                    "models", "parallel", "kernels", "backends", "support", "cli", "emulation")


_PRELOADED = set()


def _preload_kernels(device) -> None:
    """Load every kernel of the native library onto ``device`` once.

    CUDA loads kernels lazily, and the first launch of a kernel may wait for kernels
    already running on the device.  When one host thread drives several ranks, a rank's
    kernel that spins on a peer could otherwise sit in front of that peer's first launch.
    """
    import torch

    dev = torch.device(device)
    if dev.type != "cuda" or not torch.cuda.is_available():
        return
    idx = dev.index if dev.index is not None else torch.cuda.current_device()
    if idx in _PRELOADED:
        return
    from . import _native

    with torch.cuda.device(idx):
        _native.call("tccl_preload_kernels")
    _PRELOADED.add(idx)


@dataclass
class TileCCLContext:
    rank: int
    world_size: int
    device: str
    backend_name: str
    backend: Any = field(repr=False, default=None)
    topology: Any = field(default=None, repr=False)
    heap: Any = field(default=None, repr=False)
    local_group: Any = field(default=None, repr=False)
    _workspace_cache: dict = field(default_factory=dict, repr=False)
    _state: dict = field(default_factory=dict, repr=False)

    # ------------------------------------------------------------------ heap
    @property
    def has_heap(self) -> bool:
        return self.heap is not None

    @property
    def heap_bases(self):
        return self.require_heap().get_heap_bases()

    def require_heap(self):
        if self.heap is None:
            raise RuntimeError(
                "this TileCCL context has no symmetric heap; pass heap_size= (or heap=) to init()")
        return self.heap

    def attach_heap(self, heap) -> "TileCCLContext":
        if heap.rank != self.rank or heap.world_size != self.world_size:
            raise ValueError(
                f"heap is for rank {heap.rank}/{heap.world_size}, context is rank "
                f"{self.rank}/{self.world_size}")
        self.heap = heap
        self.device = str(heap.device)
        if getattr(heap, "local_group", None) is not None:
            self.local_group = heap.local_group
        self._drop_heap_state()
        if hasattr(heap, "register_reset_hook"):
            heap.register_reset_hook(self._drop_heap_state)
        _preload_kernels(heap.device)
        return self

    def _drop_heap_state(self) -> None:
        """Forget everything that points into the heap: named workspaces, the fused
        operators' signal blocks / staging / native plans / epochs, cached collective
        plans.  Runs when a heap is attached and when its allocator is reset."""
        for st in self._state.get("ops", {}).values():
            plan = st.get("plan") if isinstance(st, dict) else None
            if plan is not None and hasattr(plan, "close"):
                plan.close()
        self._workspace_cache.clear()
        self._state.clear()
        self.__dict__.pop("_collective_plans", None)

    @property
    def torch_device(self):
        import torch

        return torch.device(self.device)

    @property
    def is_single_process(self) -> bool:
        return self.local_group is not None or self.world_size == 1

    @property
    def emulated(self) -> bool:
        """True when this rank shares its GPU with another rank of the same process."""
        return self.local_group is not None and self.local_group.emulated

    def barrier(self) -> None:
        if self.heap is not None:
            self.heap.barrier()
        else:
            import torch

            torch.cuda.synchronize(self.torch_device)

    # ------------------------------------------------------------ allocators
    def allocate_tensor(self, shape, dtype):
        return self.require_heap().allocate_tensor(tuple(shape), dtype)

    def is_symmetric(self, tensor) -> bool:
        return self.heap is not None and self.heap.owns_tensor(tensor)

    def as_symmetric(self, tensor):
        return self.require_heap().as_symmetric(tensor)

    def empty(self, *size, dtype):
        return self.allocate_tensor(_normalize_size(size), dtype)

    def zeros(self, *size, dtype):
        """Zero tensor on the heap.  Fresh heap memory is zero already (no memset is issued,
        so a peer that writes into it early cannot be wiped out); see
        ``SymmetricHeap.allocate_zeroed``."""
        return self.require_heap().allocate_zeroed(_normalize_size(size), dtype)

    def randn(self, *size, dtype):
        import torch

        t = self.empty(*size, dtype=dtype)
        # Draw in fp32 on the device, then cast: same distribution for every dtype.
        t.copy_(torch.randn(t.shape, device=t.device, dtype=torch.float32))
        return t

    def workspace(self, name: str, *size, dtype, zero: bool = False):
        """A named heap tensor that is allocated once and then reused."""
        shape = _normalize_size(size)
        key = (name, shape, str(dtype))
        t = self._workspace_cache.get(key)
        if t is None:
            t = self.require_heap().allocate_zeroed(shape, dtype)
            self._workspace_cache[key] = t
        elif zero:
            t.zero_()
        return t

    # ------------------------------------------------------------ policy/info
    def auto_select_pattern(self, op: str, M: int, N: int, K: int, *, hw_info=None):
        from .patterns.auto_select import auto_select

        return auto_select(op, M, N, K, world_size=self.world_size, ctx=self, hw_info=hw_info)

    def support_matrix(self):
        from .support import describe_runtime_support

        return describe_runtime_support(self)

    def heap_metadata(self) -> dict:
        return self.require_heap().metadata()

    def runtime_metadata(self) -> dict:
        return {
            "rank": self.rank,
            "world_size": self.world_size,
            "device": self.device,
            "backend": self.backend_name,
            "has_heap": self.has_heap,
            "single_process": self.is_single_process,
            "emulated_ranks": self.emulated,
            "heap": self.heap.metadata() if self.heap is not None else None,
            "topology": self.topology.to_dict() if self.topology is not None else None,
            "config": _runtime_config_dict(),
        }


def _runtime_config_dict() -> dict:
    from .utils.config import RuntimeConfig

    return RuntimeConfig.from_env().to_dict()


def _normalize_size(size) -> tuple:
    if len(size) == 1 and isinstance(size[0], (tuple, list)):
        size = tuple(size[0])
    return tuple(int(s) for s in size)


def _resolve_backend_name(backend: str) -> str:
    name = (backend or "auto").lower()
    if name == "hip":
        raise ValueError("backend 'hip' is not available: this library targets NVIDIA B200 (CUDA) only")
    if name not in ("auto", "cuda"):
        raise ValueError(f"unknown backend {backend!r}; expected 'auto' or 'cuda'")
    return "cuda"


def _resolve_rank_world(rank, world_size) -> tuple:
    if rank is None or world_size is None:
        env_rank, env_ws = os.environ.get("RANK"), os.environ.get("WORLD_SIZE")
        dist_rank = dist_ws = None
        try:
            import torch.distributed as dist

            if dist.is_available() and dist.is_initialized():
                dist_rank, dist_ws = dist.get_rank(), dist.get_world_size()
        except Exception:
            pass
        if rank is None:
            rank = dist_rank if dist_rank is not None else int(env_rank) if env_rank else 0
        if world_size is None:
            world_size = dist_ws if dist_ws is not None else int(env_ws) if env_ws else 1
    if world_size < 1:
        raise ValueError(f"world_size must be >= 1, got {world_size}")
    if not 0 <= rank < world_size:
        raise ValueError(f"rank={rank} out of range for world_size={world_size}")
    return int(rank), int(world_size)


def _safe_topology(backend_obj):
    try:
        return backend_obj.detect_topology()
    except Exception:
        return None


def _build_context(backend: str, rank: int, world_size: int, force_backend: bool,
                   device: Optional[str] = None) -> TileCCLContext:
    from .backends import get_backend

    name = _resolve_backend_name(backend)
    backend_obj = get_backend(name, force=force_backend)
    if device is None:
        local_rank = int(os.environ.get("LOCAL_RANK", rank))
        try:
            import torch

            ndev = torch.cuda.device_count()
            device = f"cuda:{local_rank % ndev}" if ndev else f"cuda:{local_rank}"
        except Exception:
            device = f"cuda:{local_rank}"
    return TileCCLContext(rank=rank, world_size=world_size, device=device, backend_name=name,
                          backend=backend_obj, topology=_safe_topology(backend_obj))


def init(backend: str = "auto", rank: Optional[int] = None, world_size: Optional[int] = None, *,
         heap=None, heap_size: Optional[int] = None, force_backend: bool = False) -> TileCCLContext:
    """Create this process's context and make it the current one.

    Rank and world size come from the arguments, else ``torch.distributed``,
    else ``RANK`` / ``WORLD_SIZE``.  With ``heap_size`` a symmetric heap is
    created (for ``world_size > 1`` this is collective and needs
    ``torch.distributed`` to be initialised); with ``heap`` an existing one is
    attached.
    """
    global _ctx
    if heap is not None and heap_size is not None:
        raise ValueError("pass either heap= or heap_size=, not both")
    rank, world_size = _resolve_rank_world(rank, world_size)
    ctx = _build_context(backend, rank, world_size, force_backend)
    if heap is not None:
        ctx.attach_heap(heap)
    elif heap_size is not None:
        import torch

        from .memory.symmetric_heap import SymmetricHeap

        dist_ready = False
        try:
            import torch.distributed as dist

            dist_ready = dist.is_available() and dist.is_initialized()
        except Exception:
            pass
        if world_size > 1 and not dist_ready:
            raise RuntimeError(
                "init(heap_size=...) with world_size > 1 needs torch.distributed to be initialised "
                "first (e.g. dist.init_process_group('nccl') under torchrun)")
        dev_index = torch.device(ctx.device).index or 0
        torch.cuda.set_device(dev_index)
        ctx.attach_heap(SymmetricHeap(int(heap_size), rank, world_size, ctx.backend_name,
                                      device=dev_index))
    _ctx = ctx
    return ctx


def init_local(world_size: int, heap_size: int, *, backend: str = "auto",
               force_backend: bool = False, devices=None) -> list:
    """One process, ``world_size`` ranks: returns one context per rank.

    Rank ``r`` uses GPU ``r % device_count`` unless ``devices`` says otherwise, so
    more ranks than GPUs is allowed (the surplus ranks are emulated on shared
    GPUs).  Does not change the current context.
    """
    if world_size < 1:
        raise ValueError(f"world_size must be >= 1, got {world_size}")
    if heap_size is None or heap_size <= 0:
        raise ValueError(f"heap_size must be positive, got {heap_size}")
    from .memory.symmetric_heap import SymmetricHeap

    name = _resolve_backend_name(backend)
    heaps = SymmetricHeap.create_all(int(heap_size), world_size, name, devices=devices)
    ctxs = []
    for r, heap in enumerate(heaps):
        ctx = _build_context(name, r, world_size, force_backend, device=str(heap.device))
        ctx.attach_heap(heap)
        ctxs.append(ctx)
    heaps[0].local_group.contexts = ctxs
    return ctxs


def current_context() -> TileCCLContext:
    if _ctx is None:
        raise RuntimeError("TileCCL has not been initialised; call tileccl.init() first")
    return _ctx


def get_rank() -> int:
    return current_context().rank


def get_world_size() -> int:
    return current_context().world_size


def describe_runtime_support(ctx: Optional[TileCCLContext] = None):
    from .support import describe_runtime_support as _describe

    return _describe(ctx)


def __getattr__(name: str):
    if name in _LAZY_SUBMODULES:
        return importlib.import_module(f"{__name__}.{name}")
    if name in ("SymmetricHeap", "Tile"):
        from .memory.symmetric_heap import SymmetricHeap

        return SymmetricHeap
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")


__all__ = ["__version__", "init", "init_local", "get_rank", "get_world_size", "current_context",
           "describe_runtime_support", "TileCCLContext", "Tile", "SymmetricHeap",
           "patterns", "ops", "planning"]
