"""Tile primitives: device-function names (documentation stubs, see
``device_api``), the host launchers of the tile collectives, and the test harness."""

from . import collectives, device_api, harness
from .collectives import (
    AllReduceExecutionSpec,
    allgather,
    allreduce,
    broadcast,
    reduce_scatter,
    resolve_allreduce_execution,
    scatter,
)
from .device_api import *  # noqa: F401,F403
from .device_api import COLLECTIVE_DEVICE, COMMUNICATION, COMPUTE, MEMORY, DevicePrimitive

__all__ = (MEMORY + COMMUNICATION + COMPUTE + COLLECTIVE_DEVICE +
           ["allreduce", "allgather", "broadcast", "scatter", "reduce_scatter",
            "resolve_allreduce_execution", "AllReduceExecutionSpec", "DevicePrimitive",
            "collectives", "device_api", "harness"])
