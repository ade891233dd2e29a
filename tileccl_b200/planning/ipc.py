"""Device primitives under their v2 names (system scope is the only scope here).

The reference duplicates its translation and signalling primitives in the v2
package with ``scope="sys"`` defaults and adds non-consuming ``tile_poll`` /
``tile_try_poll`` (tileccl_v2/ipc.py:18-254).  In this library there is one set of
CUDA device functions (``csrc/device/symm_ptr.cuh``, ``tile_sync.cuh``), always at
system scope; these are their names.
"""

from ..primitives.device_api import (  # noqa: F401
    remote_load,
    remote_store,
    tile_poll,
    tile_signal,
    tile_signal_add,
    tile_try_poll,
    tile_try_wait,
    tile_wait,
    tile_wait_ge,
    translate_ptr,
)

remote_load_block = remote_load
remote_store_block = remote_store

__all__ = ["translate_ptr", "remote_load", "remote_store", "remote_load_block",
           "remote_store_block", "tile_signal", "tile_wait", "tile_try_wait", "tile_poll",
           "tile_try_poll", "tile_signal_add", "tile_wait_ge"]
