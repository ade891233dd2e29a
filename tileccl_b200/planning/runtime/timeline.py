"""Timeline of what ran when: spans and markers on named lanes, serialised as
JSON (schema ``tileccl.timeline.v1``, as the reference's recorder writes it,
tileccl_v2/runtime/timeline.py:86-213) and optionally drawn as a PNG.

Events come from real measurements only: CUDA-event timings, or the
``%globaltimer`` stamps kernels write into trace buffers
(:func:`events_from_device_trace`).
"""

from __future__ import annotations

import json
import math
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Iterable, Mapping, Optional, Sequence

SCHEMA = "tileccl.timeline.v1"

_CATEGORY_COLORS = {
    "producer": "#4c78a8", "ingress": "#b279a2", "frontier": "#f58518", "compute": "#54a24b",
    "aggregation": "#e45756", "marker": "#333333", "span": "#72b7b2", "comm": "#b279a2",
}


@dataclass(frozen=True)
class TimelineEvent:
    name: str
    lane: str
    start_ms: float
    end_ms: float
    category: str = "span"
    rank: Optional[int] = None
    label: Optional[str] = None
    source: str = "runtime"
    tile_range: Optional[Mapping[str, Any]] = None
    color: Optional[str] = None
    metadata: Mapping[str, Any] = field(default_factory=dict)

    def __post_init__(self) -> None:
        s, e = float(self.start_ms), float(self.end_ms)
        if not (math.isfinite(s) and math.isfinite(e)):
            raise ValueError("TimelineEvent times must be finite")
        if e < s:
            raise ValueError(f"TimelineEvent {self.name!r} has end_ms < start_ms: {e} < {s}")
        if not self.source:
            raise ValueError("TimelineEvent source must not be empty")
        object.__setattr__(self, "start_ms", s)
        object.__setattr__(self, "end_ms", e)

    @property
    def duration_ms(self) -> float:
        return self.end_ms - self.start_ms

    def to_json(self) -> dict:
        out = {"name": self.name, "lane": self.lane, "start_ms": self.start_ms,
               "end_ms": self.end_ms, "duration_ms": self.duration_ms, "category": self.category,
               "source": self.source}
        for key in ("rank", "label", "color"):
            if getattr(self, key) is not None:
                out[key] = getattr(self, key)
        if self.tile_range is not None:
            out["tile_range"] = dict(self.tile_range)
        if self.metadata:
            out["metadata"] = dict(self.metadata)
        return out

    @classmethod
    def from_json(cls, payload: Mapping[str, Any]) -> "TimelineEvent":
        return cls(name=str(payload["name"]), lane=str(payload["lane"]),
                   start_ms=float(payload["start_ms"]), end_ms=float(payload["end_ms"]),
                   category=str(payload.get("category", "span")), rank=payload.get("rank"),
                   label=payload.get("label"), source=str(payload.get("source", "runtime")),
                   tile_range=payload.get("tile_range"), color=payload.get("color"),
                   metadata=payload.get("metadata", {}))


class TimelineRecorder:
    def __init__(self, *, benchmark: str, path_name: str,
                 metadata: Optional[Mapping[str, Any]] = None) -> None:
        self.benchmark = benchmark
        self.path_name = path_name
        self.metadata = dict(metadata or {})
        self._events: list = []

    @property
    def events(self) -> tuple:
        return tuple(self._events)

    def record_span(self, *, name: str, lane: str, start_ms: float, end_ms: float,
                    category: str = "span", rank: Optional[int] = None,
                    label: Optional[str] = None, source: str = "runtime",
                    tile_range: Optional[Mapping[str, Any]] = None, color: Optional[str] = None,
                    metadata: Optional[Mapping[str, Any]] = None) -> TimelineEvent:
        ev = TimelineEvent(name, lane, start_ms, end_ms, category, rank, label, source, tile_range,
                           color, metadata or {})
        self._events.append(ev)
        return ev

    def record_marker(self, *, name: str, lane: str, at_ms: float, category: str = "marker",
                      **kwargs) -> TimelineEvent:
        return self.record_span(name=name, lane=lane, start_ms=at_ms, end_ms=at_ms,
                                category=category, **kwargs)

    def extend(self, events: Iterable[TimelineEvent]) -> None:
        self._events.extend(events)

    def lane_order(self) -> list:
        lanes: list = []
        for ev in self._events:
            if ev.lane not in lanes:
                lanes.append(ev.lane)
        return lanes

    def to_payload(self) -> dict:
        return {
            "schema": SCHEMA,
            "benchmark": self.benchmark,
            "path_name": self.path_name,
            "metadata": self.metadata,
            "lane_order": self.lane_order(),
            "events": [ev.to_json() for ev in self._events],
            "authenticity_checks": {
                "event_count": len(self._events),
                "all_events_have_source": all(bool(ev.source) for ev in self._events),
                "all_events_have_nonnegative_duration": all(ev.end_ms >= ev.start_ms
                                                            for ev in self._events),
            },
        }

    @classmethod
    def from_payload(cls, payload: Mapping[str, Any]) -> "TimelineRecorder":
        rec = cls(benchmark=str(payload["benchmark"]), path_name=str(payload["path_name"]),
                  metadata=payload.get("metadata", {}))
        rec._events.extend(TimelineEvent.from_json(p) for p in payload.get("events", []))
        return rec

    def write_json(self, path) -> None:
        path = Path(path)
        path.parent.mkdir(parents=True, exist_ok=True)
        path.write_text(json.dumps(self.to_payload(), indent=2), encoding="utf-8")

    def render_png(self, path, *, title: Optional[str] = None,
                   lane_order: Optional[Sequence[str]] = None) -> None:
        render_timeline_png(self._events, Path(path),
                            title=title or f"{self.benchmark}: {self.path_name}",
                            lane_order=lane_order)


def events_from_device_trace(done_ns: Sequence[int], *, lane: str, rank: Optional[int] = None,
                             start_ns: Optional[int] = None, name: str = "tile",
                             category: str = "compute") -> list:
    """Turn per-tile completion stamps (``%globaltimer`` nanoseconds, 0 = never ran) into
    markers relative to ``start_ns`` (default: the earliest stamp)."""
    stamps = [(i, int(t)) for i, t in enumerate(done_ns) if int(t) != 0]
    if not stamps:
        return []
    origin = int(start_ns) if start_ns is not None else min(t for _, t in stamps)
    return [TimelineEvent(f"{name}{i}", lane, (t - origin) / 1e6, (t - origin) / 1e6,
                          category="marker" if category == "marker" else category, rank=rank,
                          source="device_globaltimer", tile_range={"tile": i})
            for i, t in stamps]


def render_timeline_png(events: Sequence[TimelineEvent], path: Path, *, title: str,
                        lane_order: Optional[Sequence[str]] = None) -> None:
    """Lane diagram (matplotlib, Agg backend: no display needed)."""
    if not events:
        raise ValueError("Cannot render an empty timeline")
    try:
        import matplotlib

        matplotlib.use("Agg")
        import matplotlib.pyplot as plt
    except ImportError as exc:  # pragma: no cover - depends on the environment
        raise RuntimeError("matplotlib is not installed; write_json() is the portable artefact") from exc
    lanes = list(lane_order) if lane_order is not None else []
    for ev in events:
        if ev.lane not in lanes:
            lanes.append(ev.lane)
    ypos = {lane: len(lanes) - i for i, lane in enumerate(lanes)}
    fig, ax = plt.subplots(figsize=(12, max(2.8, 0.55 * len(lanes) + 1.6)))
    for ev in events:
        y = ypos[ev.lane]
        color = ev.color or _CATEGORY_COLORS.get(ev.category, "#72b7b2")
        if ev.duration_ms == 0:
            ax.vlines(ev.start_ms, y - 0.25, y + 0.25, color=color, linewidth=1.2)
        else:
            ax.barh(y, ev.duration_ms, left=ev.start_ms, height=0.5, color=color, alpha=0.9)
        if ev.label:
            ax.text(ev.start_ms + ev.duration_ms / 2, y + 0.3, ev.label, fontsize=7, ha="center")
    ax.set_yticks([ypos[lane] for lane in lanes])
    ax.set_yticklabels(lanes)
    ax.set_xlabel("time (ms)")
    ax.set_title(title)
    ax.grid(axis="x", alpha=0.3)
    path.parent.mkdir(parents=True, exist_ok=True)
    fig.tight_layout()
    fig.savefig(path, dpi=130)
    plt.close(fig)
