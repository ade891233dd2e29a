"""Synchronisation primitives (device functions in ``csrc/device/tile_sync.cuh``).

Same export list as the reference's ``tileccl.sync`` (tileccl/sync/__init__.py:31-51)
plus the non-consuming ``tile_poll`` / ``tile_try_poll`` of its v2 package
(tileccl_v2/ipc.py:136-254)."""

from ..primitives.device_api import (  # noqa: F401
    SYNC,
    tile_acquire_credit,
    tile_atomic_add,
    tile_atomic_and,
    tile_atomic_cas,
    tile_atomic_max,
    tile_atomic_min,
    tile_atomic_or,
    tile_atomic_xchg,
    tile_atomic_xor,
    tile_barrier,
    tile_poll,
    tile_release_credit,
    tile_signal,
    tile_signal_add,
    tile_try_poll,
    tile_try_wait,
    tile_wait,
    tile_wait_ge,
)

__all__ = list(SYNC)
