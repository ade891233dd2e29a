"""Timing and overlap analytics.

Class names follow the reference (tileccl/utils/profiling.py:20-535); the clocks
do not: ``TileProfiler`` times with CUDA events on the current stream (the
reference uses host ``perf_counter``), ``device_time_ms`` returns the max over
ranks, and the Triton-Proton wrapper becomes ``KernelProfiler``, an NVTX range
marker (NVTX ranges show up in ``ncu`` / Nsight captures; no tracing compiler is
involved here).
"""

from __future__ import annotations

import json
import time
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Callable, Optional


class TileProfiler:
    """``with TileProfiler("name") as p: ...`` - device time of the enclosed launches."""

    def __init__(self, name: str = "kernel", use_cuda_events: Optional[bool] = None) -> None:
        self.name = name
        self._use_events = use_cuda_events
        self._samples: list = []
        self._start = None
        self._end = None
        self._t0 = 0.0

    def _events_ok(self) -> bool:
        if self._use_events is not None:
            return self._use_events
        try:
            import torch

            return torch.cuda.is_available()
        except Exception:
            return False

    def __enter__(self) -> "TileProfiler":
        if self._events_ok():
            import torch

            self._start = torch.cuda.Event(enable_timing=True)
            self._end = torch.cuda.Event(enable_timing=True)
            self._start.record()
        else:
            self._start = self._end = None
            self._t0 = time.perf_counter()
        return self

    def __exit__(self, *exc: Any) -> None:
        if self._start is not None:
            self._end.record()
            self._end.synchronize()
            self._samples.append(self._start.elapsed_time(self._end))
        else:
            self._samples.append((time.perf_counter() - self._t0) * 1e3)

    @property
    def elapsed_ms(self) -> float:
        return self._samples[-1] if self._samples else 0.0

    def summary(self) -> dict:
        n = len(self._samples)
        if n == 0:
            return {"name": self.name, "count": 0}
        s = sorted(self._samples)
        return {"name": self.name, "count": n, "mean_ms": sum(s) / n, "min_ms": s[0],
                "max_ms": s[-1], "median_ms": s[n // 2],
                "clock": "cuda_events" if self._events_ok() else "host"}

    def reset(self) -> None:
        self._samples.clear()


def device_time_ms(fn: Callable[[], None], *, warmup: int = 3, iters: int = 10,
                   flush_l2_bytes: int = 0, group=None) -> float:
    """Mean device time of ``fn`` (CUDA events, optional L2 flush between iterations),
    reduced with MAX over the ranks of ``torch.distributed`` when it is initialised."""
    import torch

    flush = (torch.empty(flush_l2_bytes, dtype=torch.uint8, device="cuda")
             if flush_l2_bytes else None)
    for _ in range(max(warmup, 0)):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        if flush is not None:
            flush.zero_()
        s = torch.cuda.Event(enable_timing=True)
        e = torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        e.synchronize()
        total += s.elapsed_time(e)
    ms = total / iters
    try:
        import torch.distributed as dist

        if dist.is_available() and dist.is_initialized():
            t = torch.tensor([ms], dtype=torch.float64, device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
            ms = float(t.item())
    except Exception:
        pass
    return ms


def bandwidth_to_normalized(bytes_transferred: float, time_ms: float,
                            peak_gbps: float = 900.0) -> dict:
    """GB/s and fraction of a peak for ``bytes_transferred`` in ``time_ms``."""
    if time_ms <= 0:
        return {"gbps": 0.0, "fraction_of_peak": 0.0, "peak_gbps": peak_gbps}
    gbps = bytes_transferred / (time_ms * 1e-3) / 1e9
    return {"gbps": gbps, "fraction_of_peak": gbps / peak_gbps if peak_gbps > 0 else 0.0,
            "peak_gbps": peak_gbps}


def format_benchmark_table(results: list) -> str:
    """Plain-text table from a list of flat dicts (columns = union of keys, in first-seen order)."""
    if not results:
        return "(no results)"
    cols: list = []
    for r in results:
        for k in r:
            if k not in cols:
                cols.append(k)

    def cell(v: Any) -> str:
        return f"{v:.4f}" if isinstance(v, float) else str(v)

    rows = [[cell(r.get(c, "")) for c in cols] for r in results]
    widths = [max(len(c), *(len(row[i]) for row in rows)) for i, c in enumerate(cols)]
    line = "  ".join(c.ljust(w) for c, w in zip(cols, widths))
    sep = "  ".join("-" * w for w in widths)
    body = ["  ".join(v.ljust(w) for v, w in zip(row, widths)) for row in rows]
    return "\n".join([line, sep, *body])


def save_benchmark_results(results: Any, path, *, metadata: Optional[dict] = None) -> Path:
    path = Path(path)
    path.parent.mkdir(parents=True, exist_ok=True)
    payload = {"results": results, "metadata": metadata or {}, "timestamp": time.time()}
    path.write_text(json.dumps(payload, indent=2, default=str))
    return path


class KernelProfiler:
    """NVTX range marker (no-op when NVTX is unavailable)."""

    def __init__(self, name: str = "tileccl_profile") -> None:
        self.name = name
        try:
            import torch

            self._nvtx = torch.cuda.nvtx if torch.cuda.is_available() else None
        except Exception:
            self._nvtx = None

    @property
    def available(self) -> bool:
        return self._nvtx is not None

    class _Range:
        def __init__(self, nvtx, name):
            self._nvtx, self._name = nvtx, name

        def __enter__(self):
            if self._nvtx is not None:
                self._nvtx.range_push(self._name)
            return self

        def __exit__(self, *exc):
            if self._nvtx is not None:
                self._nvtx.range_pop()

    def session(self, label: Optional[str] = None) -> "KernelProfiler._Range":
        return KernelProfiler._Range(self._nvtx, label or self.name)

    def export(self, path) -> None:
        """Ranges are consumed by the external profiler; this writes a marker file naming them."""
        Path(path).write_text(json.dumps({"profiler": "nvtx", "range": self.name}))


ProtonProfiler = KernelProfiler  # name used by code written against the reference


@dataclass
class _Interval:
    stream: str
    name: str
    start_ms: float
    end_ms: float


class OverlapTimeline:
    """How much of the communication time was hidden under computation."""

    def __init__(self) -> None:
        self._events: list = []

    def record(self, stream: str, name: str, start_ms: float, end_ms: float) -> None:
        if end_ms < start_ms:
            raise ValueError(f"interval {name!r} ends before it starts")
        if stream not in ("compute", "comm"):
            raise ValueError("stream must be 'compute' or 'comm'")
        self._events.append(_Interval(stream, name, float(start_ms), float(end_ms)))

    @staticmethod
    def _union(intervals: list) -> list:
        merged: list = []
        for s, e in sorted(intervals):
            if merged and s <= merged[-1][1]:
                merged[-1][1] = max(merged[-1][1], e)
            else:
                merged.append([s, e])
        return merged

    def compute_overlap(self) -> dict:
        comp = self._union([(e.start_ms, e.end_ms) for e in self._events if e.stream == "compute"])
        comm = self._union([(e.start_ms, e.end_ms) for e in self._events if e.stream == "comm"])
        total_comp = sum(e - s for s, e in comp)
        total_comm = sum(e - s for s, e in comm)
        overlap, i, j = 0.0, 0, 0
        while i < len(comp) and j < len(comm):
            lo, hi = max(comp[i][0], comm[j][0]), min(comp[i][1], comm[j][1])
            if hi > lo:
                overlap += hi - lo
            if comp[i][1] < comm[j][1]:
                i += 1
            else:
                j += 1
        spans = comp + comm
        wall = (max(e for _, e in spans) - min(s for s, _ in spans)) if spans else 0.0
        serial = total_comp + total_comm
        return {"compute_ms": total_comp, "comm_ms": total_comm, "overlap_ms": overlap,
                "overlap_ratio": overlap / total_comm if total_comm > 0 else 0.0,
                "wall_ms": wall, "efficiency": serial / wall if wall > 0 else 0.0}

    def export_json(self, path) -> None:
        Path(path).write_text(json.dumps(
            {"events": [e.__dict__ for e in self._events], "overlap": self.compute_overlap()},
            indent=2))

    def print_summary(self) -> None:
        o = self.compute_overlap()
        print(f"compute {o['compute_ms']:.3f} ms, comm {o['comm_ms']:.3f} ms, overlapped "
              f"{o['overlap_ms']:.3f} ms ({o['overlap_ratio']:.1%} of comm), wall {o['wall_ms']:.3f} ms")


class CommHeatmap:
    """src x dst matrix of bytes and message counts."""

    def __init__(self, world_size: int) -> None:
        if world_size < 1:
            raise ValueError("world_size must be >= 1")
        self.world_size = world_size
        self._bytes = [[0] * world_size for _ in range(world_size)]
        self._count = [[0] * world_size for _ in range(world_size)]

    def record(self, src: int, dst: int, bytes_transferred: int) -> None:
        for name, r in (("src", src), ("dst", dst)):
            if not 0 <= r < self.world_size:
                raise ValueError(f"{name}={r} out of range for world_size={self.world_size}")
        self._bytes[src][dst] += int(bytes_transferred)
        self._count[src][dst] += 1

    def get_traffic_matrix(self) -> list:
        return [row[:] for row in self._bytes]

    def get_count_matrix(self) -> list:
        return [row[:] for row in self._count]

    def balance(self) -> dict:
        sent = [sum(row) for row in self._bytes]
        hi, lo = max(sent), min(sent)
        return {"max_send_bytes": hi, "min_send_bytes": lo,
                "max_min_send_ratio": hi / lo if lo > 0 else float("inf") if hi > 0 else 1.0}

    def print_matrix(self, unit: str = "MB") -> None:
        div = {"B": 1, "KB": 1e3, "MB": 1e6, "GB": 1e9}[unit]
        print("src\\dst " + " ".join(f"{d:>10d}" for d in range(self.world_size)))
        for s, row in enumerate(self._bytes):
            print(f"{s:>7d} " + " ".join(f"{v / div:>10.2f}" for v in row))

    def export_json(self, path) -> None:
        Path(path).write_text(json.dumps({"world_size": self.world_size, "bytes": self._bytes,
                                          "counts": self._count, "balance": self.balance()},
                                         indent=2))
