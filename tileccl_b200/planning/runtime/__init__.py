"""Runtime observability helpers of the planning package."""

from .timeline import (SCHEMA, TimelineEvent, TimelineRecorder, events_from_device_trace,
                       render_timeline_png, render_timeline_svg)

__all__ = ["SCHEMA", "TimelineEvent", "TimelineRecorder", "events_from_device_trace",
           "render_timeline_png", "render_timeline_svg"]
