"""Topology helpers with the reference's function names (tileccl/utils/topology.py:22-246),
answered by the native device query.  (The reference reads ``props.total_mem``,
which current PyTorch does not have, so its detection silently yields nothing;
and it labels B200's NV18 links plain "NVLink".)
"""

from __future__ import annotations

from ..backends import TopologyInfo, detect_hardware, get_backend

__all__ = ["TopologyInfo", "TopologyDetector", "detect_backend", "detect_topology",
           "get_num_compute_units", "get_warp_size", "get_optimal_num_sms", "print_topology_info"]

B200_SMS = 148


def detect_backend() -> str:
    """``"cuda"`` or ``"none"``."""
    return detect_hardware()


def detect_topology(backend: str = "auto") -> TopologyInfo:
    if detect_hardware() != "cuda":
        return TopologyInfo(num_gpus=0, link_type="none")
    return get_backend(backend).detect_topology()


def get_num_compute_units(backend: str = "auto") -> int:
    if detect_hardware() != "cuda":
        return B200_SMS
    return get_backend(backend).get_device_properties(0).compute_units


def get_warp_size(backend: str = "auto") -> int:
    return 32


def get_optimal_num_sms(backend: str = "auto") -> int:
    """Grid of a persistent kernel: one CTA per SM."""
    return get_num_compute_units(backend)


def print_topology_info(info: TopologyInfo) -> None:
    print(f"GPUs: {info.num_gpus}  link: {info.link_type}"
          + (f" (NVLink {info.nvlink_generation}, {info.links_per_gpu} links/GPU)"
             if info.nvlink_generation else ""))
    print(f"bandwidth per direction per GPU: {info.bandwidth_gbps:.0f} GB/s  "
          f"fully connected: {info.is_fully_connected}  NVLS multicast: {info.multicast_supported}")
    print(f"SMs: {info.num_compute_units}")
    for i, row in enumerate(info.peer_access_matrix):
        print(f"  gpu{i}: " + " ".join("P" if ok else "-" for ok in row))


class TopologyDetector:
    def detect(self, backend: str = "auto") -> TopologyInfo:
        return detect_topology(backend)

    @staticmethod
    def print_info(info: TopologyInfo) -> None:
        print_topology_info(info)
