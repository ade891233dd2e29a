"""Debug build: device-side bounds checks that record instead of trapping.

The reference has no sanitizer of its own: its safety rests on the protocol
(release/acquire at system scope, monotonic epochs; tileccl/primitives/collectives.py:348-352).
Here a second build of the native library (``python -m tileccl_b200._build --debug``,
loaded when ``TILECCL_DEBUG=1``) compiles the device primitives with
``-DTILECCL_DEBUG_CHECKS``: every pointer translation and every symmetric tile or span a
verb or a collective is about to touch is checked against the heap window.  A violation is
written to a per-device record (first offender wins, a counter keeps counting), the access
is redirected to the caller's own copy or skipped, and the kernel runs to its end, so the
context stays usable and no GPU faults.  This module reads the records, and
``after_collective`` is the per-call check the collective launchers run in debug mode:
status words, bounds records and the epoch invariants of the counter block.
"""

from __future__ import annotations

import ctypes as C
from typing import List, Optional

from . import _native
from .utils.config import current as _config

CODES = {
    1: "rank outside [0, world_size)",
    2: "address not inside the owner's heap",
    3: "span leaves the owner's heap",
    4: "multimem verb without a bound multicast mapping",
}


class DebugRecord(C.Structure):
    """Mirror of ``tileccl::DebugRecord`` (csrc/device/symm_ptr.cuh)."""

    _fields_ = [("count", C.c_uint32), ("code", C.c_uint32), ("rank", C.c_int32),
                ("from_rank", C.c_int32), ("to_rank", C.c_int32), ("enabled", C.c_uint32),
                ("addr", C.c_uint64), ("bytes", C.c_uint64)]

    def to_dict(self, source: str) -> dict:
        return {"source": source, "count": int(self.count), "code": int(self.code),
                "what": CODES.get(int(self.code), "unknown"), "rank": int(self.rank),
                "owner_rank": int(self.from_rank), "to_rank": int(self.to_rank),
                "addr": int(self.addr), "bytes": int(self.bytes)}


class TileCCLDebugError(RuntimeError):
    """A device-side bounds check of the debug build recorded a violation."""


_READERS = (("primitives", "tccl_debug_read_primitives"),
            ("collectives", "tccl_debug_read_collectives"))


def is_debug_build() -> bool:
    """True when the loaded native library was compiled with the recorded bounds checks."""
    rec = DebugRecord()
    _native.call("tccl_debug_read_primitives", C.byref(rec), 0)
    return bool(rec.enabled)


def read_records(device=None, *, clear: bool = True, user_modules=()) -> List[dict]:
    """Violations recorded on ``device`` (default: the current one) since the last clear.

    Synchronises the device first, so everything launched before the call has been
    checked.  ``user_modules``: ``userkernel.UserKernelModule`` objects compiled with
    ``debug=True`` whose records should be read as well."""
    import torch

    out: List[dict] = []
    with torch.cuda.device(device if device is not None else torch.cuda.current_device()):
        torch.cuda.synchronize()
        for source, fn in _READERS:
            rec = DebugRecord()
            _native.call(fn, C.byref(rec), 1 if clear else 0)
            if rec.count:
                out.append(rec.to_dict(source))
        for mod in user_modules:
            rec = mod.debug_record(clear=clear)
            if rec is not None and rec.count:
                out.append(rec.to_dict(f"user:{mod.path.name}"))
    return out


def check(device=None, *, user_modules=()) -> None:
    """Raise :class:`TileCCLDebugError` if a bounds check recorded a violation."""
    recs = read_records(device, user_modules=user_modules)
    if recs:
        r = recs[0]
        raise TileCCLDebugError(
            f"{sum(x['count'] for x in recs)} bounds violation(s); first ({r['source']}): "
            f"{r['what']}: rank {r['rank']}, owner {r['owner_rank']}, to_rank {r['to_rank']}, "
            f"address {r['addr']:#x}, {r['bytes']} bytes")


def epoch_invariant_errors(counters, epoch: int, rank: int, world_size: int,
                           root: Optional[int] = None) -> List[str]:
    """Check a collective counter block (``ready[0:8]``, ``done[8:16]``, host list of ints)
    after call number ``epoch`` has completed on this rank.

    Counters only grow, by one per call and source.  Once this rank's kernel has returned,
    every source it depends on has announced and completed call ``epoch``; a faster peer may
    already have announced call ``epoch + 1`` but cannot have completed it (its data phase
    waits for this rank's announcement).  Rooted calls only move the counters between the
    root and the others."""
    errs = []
    for src in range(world_size):
        if src == rank:
            continue
        ready, done = int(counters[src]), int(counters[8 + src])
        if root is None:
            dep_ready, dep_done = True, True
        else:
            dep_ready, dep_done = (rank == root), (src == root)
        if dep_ready and not epoch <= ready <= epoch + 1:
            errs.append(f"ready[{src}] = {ready}, expected {epoch} or {epoch + 1}")
        if dep_done and not epoch <= done <= epoch + 1:
            errs.append(f"done[{src}] = {done}, expected {epoch} or {epoch + 1}")
        if not dep_ready and ready != 0 and root is not None and rank != root:
            errs.append(f"ready[{src}] = {ready} on a non-root rank of a rooted call")
    return errs


def after_collective(heap, state: dict, epoch: int, *, root: Optional[int] = None) -> None:
    """Debug-mode epilogue of one collective call on a one-process-per-GPU heap: wait for the
    kernel, raise on a timed-out wait, on a recorded bounds violation and on a counter block
    that breaks the epoch invariants."""
    import torch

    from .kernels.fused_gemm import raise_on_status

    torch.cuda.synchronize(heap.device)
    status = heap._state.get("status")
    if status is not None:
        raise_on_status(status)
    if is_debug_build():
        check(heap.device)
    errs = epoch_invariant_errors(state["counters"].tolist(), epoch, heap.rank, heap.world_size,
                                  root)
    if errs:
        raise TileCCLDebugError(f"collective epoch {epoch} on rank {heap.rank}: " + "; ".join(errs))


def enabled() -> bool:
    """``TILECCL_DEBUG`` is set (the collective launchers then call :func:`after_collective`)."""
    return _config().debug
