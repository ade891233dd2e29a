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

# Colours of the categories this library's own traces use; anything else gets a hue
# derived from the category name (see _colour_of).
_CATEGORY_COLORS = {
    "compute": "#2e7d32", "mma": "#1b5e20", "epilogue": "#1565c0", "push": "#ef6c00",
    "comm": "#ef6c00", "wait": "#9e9e9e", "signal": "#6a1b9a", "copy": "#00838f",
    "marker": "#212121", "span": "#546e7a",
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

    def render_svg(self, path, *, title: Optional[str] = None,
                   lane_order: Optional[Sequence[str]] = None) -> None:
        render_timeline_svg(self._events, Path(path),
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


def _lanes_of(events: Sequence[TimelineEvent], lane_order: Optional[Sequence[str]]) -> list:
    lanes = list(lane_order) if lane_order is not None else []
    for ev in events:
        if ev.lane not in lanes:
            lanes.append(ev.lane)
    return lanes


def _colour_of(ev: TimelineEvent) -> str:
    if ev.color:
        return ev.color
    known = _CATEGORY_COLORS.get(ev.category)
    if known:
        return known
    # categories without an entry get a stable hue derived from their name
    hue = sum(ord(ch) * (i + 7) for i, ch in enumerate(ev.category)) % 360
    return f"hsl({hue}, 55%, 48%)"


def render_timeline_svg(events: Sequence[TimelineEvent], path: Path, *, title: str,
                        lane_order: Optional[Sequence[str]] = None, width: int = 1200) -> None:
    """Lane diagram as a stand-alone SVG file, written with nothing but the standard library
    (one row per lane, one rectangle per span, one tick per marker, a time axis in ms)."""
    if not events:
        raise ValueError("Cannot render an empty timeline")
    from xml.sax.saxutils import escape

    lanes = _lanes_of(events, lane_order)
    t0 = min(ev.start_ms for ev in events)
    t1 = max(ev.end_ms for ev in events)
    span = max(t1 - t0, 1e-9)
    label_w = 12 + 7 * max(len(lane) for lane in lanes)
    row_h, top, bottom = 26, 44, 40
    plot_w = max(200, width - label_w - 24)
    height = top + row_h * len(lanes) + bottom

    def x_of(t_ms: float) -> float:
        return label_w + (t_ms - t0) / span * plot_w

    out = [f'<svg xmlns="http://www.w3.org/2000/svg" width="{width}" height="{height}" '
           f'font-family="monospace" font-size="11">',
           f'<rect width="{width}" height="{height}" fill="white"/>',
           f'<text x="{label_w}" y="20" font-size="14">{escape(title)}</text>']
    for i, lane in enumerate(lanes):
        y = top + i * row_h
        shade = "#f4f4f4" if i % 2 == 0 else "#ffffff"
        out.append(f'<rect x="{label_w}" y="{y}" width="{plot_w}" height="{row_h}" fill="{shade}"/>')
        out.append(f'<text x="{label_w - 6}" y="{y + row_h * 0.65:.1f}" text-anchor="end">'
                   f'{escape(lane)}</text>')
    row = {lane: i for i, lane in enumerate(lanes)}
    for ev in events:
        y = top + row[ev.lane] * row_h
        colour = _colour_of(ev)
        tip = f"{ev.name} [{ev.category}] {ev.start_ms:.4f}-{ev.end_ms:.4f} ms"
        if ev.end_ms > ev.start_ms:
            w_px = max(0.5, x_of(ev.end_ms) - x_of(ev.start_ms))
            out.append(f'<rect x="{x_of(ev.start_ms):.2f}" y="{y + 4}" width="{w_px:.2f}" '
                       f'height="{row_h - 8}" fill="{colour}"><title>{escape(tip)}</title></rect>')
        else:
            x = x_of(ev.start_ms)
            out.append(f'<line x1="{x:.2f}" x2="{x:.2f}" y1="{y + 2}" y2="{y + row_h - 2}" '
                       f'stroke="{colour}" stroke-width="1.5"><title>{escape(tip)}</title></line>')
        if ev.label:
            out.append(f'<text x="{x_of((ev.start_ms + ev.end_ms) / 2):.2f}" y="{y + 3}" '
                       f'text-anchor="middle" font-size="9">{escape(ev.label)}</text>')
    axis_y = top + row_h * len(lanes)
    for k in range(11):
        t = t0 + span * k / 10
        x = x_of(t)
        out.append(f'<line x1="{x:.2f}" x2="{x:.2f}" y1="{top}" y2="{axis_y + 4}" stroke="#bbbbbb" '
                   f'stroke-width="0.5"/>')
        out.append(f'<text x="{x:.2f}" y="{axis_y + 18}" text-anchor="middle">{t:.3f}</text>')
    out.append(f'<text x="{label_w + plot_w / 2:.1f}" y="{axis_y + 34}" text-anchor="middle">'
               f'time (ms)</text></svg>')
    path = Path(path)
    path.parent.mkdir(parents=True, exist_ok=True)
    path.write_text("\n".join(out), encoding="utf-8")


def render_timeline_png(events: Sequence[TimelineEvent], path: Path, *, title: str,
                        lane_order: Optional[Sequence[str]] = None) -> None:
    """Raster version of :func:`render_timeline_svg` for callers that ask for a PNG (needs
    matplotlib, headless Agg canvas).  Spans of one lane and colour are drawn as one
    ``broken_barh`` collection, markers as one event plot per lane."""
    if not events:
        raise ValueError("Cannot render an empty timeline")
    try:
        from matplotlib.backends.backend_agg import FigureCanvasAgg
        from matplotlib.figure import Figure
    except ImportError as exc:  # pragma: no cover - depends on the environment
        raise RuntimeError("matplotlib is not installed; write_json() and render_svg() need "
                           "nothing beyond the standard library") from exc
    lanes = _lanes_of(events, lane_order)
    fig = Figure(figsize=(11.5, 1.2 + 0.4 * len(lanes)), dpi=120)
    FigureCanvasAgg(fig)
    ax = fig.add_subplot(111)
    for row, lane in enumerate(lanes):
        mine = [ev for ev in events if ev.lane == lane]
        by_colour: dict = {}
        for ev in mine:
            if ev.end_ms > ev.start_ms:
                by_colour.setdefault(_colour_of(ev), []).append((ev.start_ms, ev.end_ms - ev.start_ms))
        for colour, spans in by_colour.items():
            ax.broken_barh(spans, (row - 0.35, 0.7), facecolors=colour if not colour.startswith("hsl")
                           else "#5f9ea0")
        ticks = [ev.start_ms for ev in mine if ev.end_ms == ev.start_ms]
        if ticks:
            ax.eventplot(ticks, lineoffsets=row, linelengths=0.7, colors="black", linewidths=0.8)
    ax.set_ylim(len(lanes) - 0.5, -0.5)          # first lane on top
    ax.set_yticks(range(len(lanes)), labels=lanes)
    ax.set_xlabel("time (ms)")
    ax.set_title(title, loc="left")
    ax.grid(True, axis="x", linewidth=0.3)
    path = Path(path)
    path.parent.mkdir(parents=True, exist_ok=True)
    fig.savefig(path, bbox_inches="tight")
