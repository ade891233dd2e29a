"""Read-only NVLink facts from NVML: how many links a GPU has up, their generation and
their line rate.  The reference probes links 0-5 only and classifies the interconnect from
``nvidia-smi topo -m`` text (tileccl/backends/cuda.py:326-372); a B200 has 18 links.

Nothing here changes a GPU setting.  ``nvml`` may be injected (tests pass a fake module).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

MAX_LINKS = 18
# NVML_NVLINK_VERSION_* -> NVLink generation
_VERSION_TO_GENERATION = {1: 1, 2: 2, 3: 2, 4: 3, 5: 3, 6: 4, 7: 5}
# per-direction payload rate of one link in GB/s, by generation (fallback when the
# speed field is not reported)
_LINK_GBPS = {1: 20.0, 2: 25.0, 3: 25.0, 4: 25.0, 5: 50.0}


@dataclass(frozen=True)
class NvlinkFacts:
    links_active: int
    generation: int
    gbps_per_direction: float     # all active links together, one direction
    source: str                   # "nvml" | "nvml-partial"

    def to_dict(self) -> dict:
        return {"links_active": self.links_active, "generation": self.generation,
                "gbps_per_direction": self.gbps_per_direction, "source": self.source}


def _load():
    try:
        import pynvml

        pynvml.nvmlInit()
        return pynvml
    except Exception:
        return None


def nvlink_facts(index: int = 0, nvml=None, uuid: Optional[str] = None) -> Optional[NvlinkFacts]:
    """Facts for GPU ``index`` (or ``uuid``); ``None`` when NVML or NVLink is unavailable."""
    n = nvml if nvml is not None else _load()
    if n is None:
        return None
    try:
        handle = (n.nvmlDeviceGetHandleByUUID(uuid.encode() if isinstance(uuid, str) else uuid)
                  if uuid else n.nvmlDeviceGetHandleByIndex(index))
    except Exception:
        return None
    active, version = 0, 0
    for link in range(MAX_LINKS):
        try:
            if int(n.nvmlDeviceGetNvLinkState(handle, link)) != 1:
                continue
        except Exception:
            break                        # link index not present on this GPU
        active += 1
        if version == 0:
            try:
                version = int(n.nvmlDeviceGetNvLinkVersion(handle, link))
            except Exception:
                version = 0
    if active == 0:
        return None
    generation = _VERSION_TO_GENERATION.get(version, 0)
    source = "nvml"
    per_link = None
    try:
        field = getattr(n, "NVML_FI_DEV_NVLINK_SPEED_MBPS_COMMON")
        vals = n.nvmlDeviceGetFieldValues(handle, [field])
        v = vals[0]
        mbps = getattr(getattr(v, "value", None), "uiVal", None)
        if getattr(v, "nvmlReturn", 0) == 0 and mbps:
            per_link = float(mbps) / 1000.0
    except Exception:
        per_link = None
    if per_link is None:
        per_link = _LINK_GBPS.get(generation, 25.0)
        source = "nvml-partial"
    return NvlinkFacts(active, generation, per_link * active, source)
