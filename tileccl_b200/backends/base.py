"""Dataclasses describing a device and the node's interconnect.

Field names follow the reference (tileccl/backends/base.py:19-69) so that code
such as ``ctx.backend.get_device_properties().compute_units`` keeps working; the
values come from the native device query, not from parsing ``nvidia-smi``.
"""

from __future__ import annotations

from dataclasses import dataclass, field


@dataclass
class TopologyInfo:
    num_gpus: int = 0
    backend: str = "cuda"
    link_type: str = "unknown"           # "NVSwitch", "NVLink", "PCIe", "none"
    nvlink_generation: int = 0
    links_per_gpu: int = 0
    peer_access_matrix: list = field(default_factory=list)
    native_atomics_matrix: list = field(default_factory=list)
    bandwidth_gbps: float = 0.0           # per direction, per GPU
    is_fully_connected: bool = False
    multicast_supported: bool = False
    num_compute_units: int = 0

    def to_dict(self) -> dict:
        return dict(self.__dict__)


@dataclass
class DeviceProperties:
    name: str = ""
    ordinal: int = 0
    compute_units: int = 0
    warp_size: int = 32
    max_shared_memory: int = 0
    total_memory: int = 0
    l2_cache_bytes: int = 0
    clock_mhz: float = 0.0
    memory_clock_mhz: float = 0.0
    memory_bus_bits: int = 0
    compute_capability: tuple = (0, 0)
    vmm_supported: bool = False
    posix_fd_handles: bool = False
    fabric_handles: bool = False
    multicast_supported: bool = False

    @property
    def arch(self) -> str:
        return f"sm_{self.compute_capability[0]}{self.compute_capability[1]}"

    def to_dict(self) -> dict:
        d = dict(self.__dict__)
        d["compute_capability"] = list(self.compute_capability)
        d["arch"] = self.arch
        return d


class BackendInterface:
    """What the rest of the library may ask of the device layer."""

    name = "base"

    def device_count(self) -> int:  # pragma: no cover - interface
        raise NotImplementedError

    def get_device_properties(self, device_id: int = 0) -> DeviceProperties:  # pragma: no cover
        raise NotImplementedError

    def detect_topology(self) -> TopologyInfo:  # pragma: no cover
        raise NotImplementedError

    def synchronize(self, device_id: int | None = None) -> None:  # pragma: no cover
        raise NotImplementedError
