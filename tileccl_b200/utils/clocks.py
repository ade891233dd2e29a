"""Read-only sampling of a GPU's SM clock and throttle reasons through NVML.

Benchmarks run a :class:`ClockSampler` thread during their timed region so that a
number taken while the GPU was throttled (or with its clocks pinned low) can be
recognised and taken again.  Nothing here changes any GPU setting.
"""

from __future__ import annotations

import statistics
import threading
import time

# NVML clocks-event-reason bits that make a measurement suspect.
_REASON_BITS = {
    0x0000000000000004: "sw_power_cap",
    0x0000000000000008: "hw_slowdown",
    0x0000000000000020: "sw_thermal_slowdown",
    0x0000000000000040: "hw_thermal_slowdown",
    0x0000000000000080: "hw_power_brake_slowdown",
}
REJECTING = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown")


class ClockSampler:
    """Samples every ``period_s`` from a background thread between start() and stop()."""

    def __init__(self, cuda_index: int = 0, period_s: float = 0.005):
        self.cuda_index = cuda_index
        self.period_s = period_s
        self._samples: list = []
        self._reasons: set = set()
        self._stop = threading.Event()
        self._thread = None
        self._handle = None
        self._nvml = None
        self._max_mhz = None
        self.error = None

    def _open(self) -> None:
        import pynvml

        pynvml.nvmlInit()
        self._nvml = pynvml
        handle = None
        try:
            import torch

            uuid = str(torch.cuda.get_device_properties(self.cuda_index).uuid)
            if not uuid.startswith("GPU-"):
                uuid = "GPU-" + uuid
            handle = pynvml.nvmlDeviceGetHandleByUUID(uuid.encode())
        except Exception:
            handle = pynvml.nvmlDeviceGetHandleByIndex(self.cuda_index)
        self._handle = handle
        self._max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(handle, pynvml.NVML_CLOCK_SM))

    def _sample(self) -> None:
        n = self._nvml
        mhz = float(n.nvmlDeviceGetClockInfo(self._handle, n.NVML_CLOCK_SM))
        try:
            power = n.nvmlDeviceGetPowerUsage(self._handle) / 1000.0
        except Exception:
            power = None
        try:
            mask = int(n.nvmlDeviceGetCurrentClocksEventReasons(self._handle))
        except Exception:
            try:
                mask = int(n.nvmlDeviceGetCurrentClocksThrottleReasons(self._handle))
            except Exception:
                mask = 0
        for bit, name in _REASON_BITS.items():
            if mask & bit:
                self._reasons.add(name)
        self._samples.append((time.perf_counter(), mhz, power))

    def _run(self) -> None:
        while not self._stop.is_set():
            try:
                self._sample()
            except Exception as exc:  # pragma: no cover - depends on the machine
                self.error = repr(exc)
                return
            self._stop.wait(self.period_s)

    def start(self) -> "ClockSampler":
        try:
            self._open()
            self._sample()
        except Exception as exc:
            self.error = repr(exc)
            return self
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()
        return self

    def stop(self) -> dict:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2.0)
            try:
                self._sample()
            except Exception:
                pass
        if not self._samples:
            return {"sm_mhz": None, "sm_max_mhz": self._max_mhz, "samples": 0,
                    "reasons": [f"nvml unavailable: {self.error}"]}
        mhz = [s[1] for s in self._samples]
        powers = [s[2] for s in self._samples if s[2] is not None]
        out = {"sm_mhz": statistics.median(mhz), "sm_min_mhz": min(mhz), "sm_max_mhz": self._max_mhz,
               "samples": len(mhz), "reasons": sorted(self._reasons)}
        if powers:
            out["power_w_max"] = max(powers)
        out["rejected"] = any(r in REJECTING for r in self._reasons)
        return out
