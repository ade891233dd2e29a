"""The one device backend: NVIDIA B200 through ``libtileccl_b200``.

The reference loads ``libcudart`` with ctypes and classifies the interconnect by
parsing ``nvidia-smi topo -m`` (tileccl/backends/cuda.py:79-187, 326-372; its
string match files B200's ``NV18`` under plain "NVLink").  Here the peer matrix,
multicast capability and SM count come from the CUDA runtime / driver, and an
all-to-all peer matrix with multicast support is reported as NVSwitch.
"""

from __future__ import annotations

import ctypes as C

from .. import _native
from .base import BackendInterface, DeviceProperties, TopologyInfo

# Fallback when NVML cannot be asked (see backends/nvml.py for the measured facts):
# per-direction, per-GPU NVLink bandwidth in GB/s by compute capability major.
_NVLINK_GBPS = {8: 300.0, 9: 450.0, 10: 900.0}
_NVLINK_GEN = {8: 3, 9: 4, 10: 5}
_NVLINK_LINKS = {8: 12, 9: 18, 10: 18}
PCIE_GBPS = 32.0


class CUDABackend(BackendInterface):
    name = "cuda"
    _nvml = None      # a module with the pynvml API; None = import pynvml on demand

    def device_count(self) -> int:
        n = C.c_int32()
        _native.call("tccl_device_count", C.byref(n))
        return int(n.value)

    def get_device_properties(self, device_id: int = 0) -> DeviceProperties:
        p = _native.DeviceProps()
        _native.call("tccl_device_props", int(device_id), C.byref(p))
        return DeviceProperties(
            name=p.name.decode(errors="replace"),
            ordinal=p.ordinal,
            compute_units=p.sm_count,
            warp_size=p.warp_size,
            max_shared_memory=p.max_smem_per_block_optin,
            total_memory=p.total_mem,
            l2_cache_bytes=p.l2_bytes,
            clock_mhz=p.clock_khz / 1000.0,
            memory_clock_mhz=p.mem_clock_khz / 1000.0,
            memory_bus_bits=p.mem_bus_bits,
            compute_capability=(p.cc_major, p.cc_minor),
            vmm_supported=bool(p.vmm_supported),
            posix_fd_handles=bool(p.posix_fd_handles),
            fabric_handles=bool(p.fabric_handles),
            multicast_supported=bool(p.multicast_supported),
        )

    def peer_matrix(self, n: int | None = None) -> tuple[list, list]:
        n = self.device_count() if n is None else n
        access = (C.c_int32 * (n * n))()
        atomics = (C.c_int32 * (n * n))()
        if n:
            _native.call("tccl_peer_matrix", n, access, atomics)
        to_rows = lambda a: [[bool(a[i * n + j]) for j in range(n)] for i in range(n)]
        return to_rows(access), to_rows(atomics)

    def detect_topology(self) -> TopologyInfo:
        n = self.device_count()
        if n == 0:
            return TopologyInfo(num_gpus=0, link_type="none")
        props = self.get_device_properties(0)
        access, atomics = self.peer_matrix(n)
        full = all(all(row) for row in access)
        mc = all(self.get_device_properties(i).multicast_supported for i in range(n))
        major = props.compute_capability[0]
        if n == 1:
            link, bw = "none", 0.0
        elif full and mc:
            link, bw = "NVSwitch", _NVLINK_GBPS.get(major, 450.0)
        elif full and all(all(r) for r in atomics):
            link, bw = "NVLink", _NVLINK_GBPS.get(major, 300.0)
        elif any(any(r[j] for j in range(n) if j != i) for i, r in enumerate(access)):
            link, bw = "PCIe", PCIE_GBPS
        else:
            link, bw = "none", 0.0
        gen = _NVLINK_GEN.get(major, 0) if link in ("NVSwitch", "NVLink") else 0
        links = _NVLINK_LINKS.get(major, 0) if link in ("NVSwitch", "NVLink") else 0
        if link in ("NVSwitch", "NVLink"):
            # Link count, generation and line rate as NVML reports them (read-only queries).
            from .nvml import nvlink_facts

            facts = nvlink_facts(0, nvml=self._nvml)
            if facts is not None:
                links = facts.links_active
                gen = facts.generation or gen
                bw = facts.gbps_per_direction or bw
        return TopologyInfo(
            num_gpus=n, backend="cuda", link_type=link,
            nvlink_generation=gen,
            links_per_gpu=links,
            peer_access_matrix=access, native_atomics_matrix=atomics, bandwidth_gbps=bw,
            is_fully_connected=full, multicast_supported=mc, num_compute_units=props.compute_units)

    def synchronize(self, device_id: int | None = None) -> None:
        import torch

        torch.cuda.synchronize(device_id)
