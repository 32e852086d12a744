"""Tag-based tracing (second generation): timelines of spans per host thread and per device."""
from .constants import *  # noqa: F401,F403
from .timeline import AsyncTimeline, BatchAsyncTimelines, Span, Timeline
from .tracer import AsyncWaitlist, NoopTracer, PerfTracer
from .export import PerfMetricsExport, log_metric_export_fn
from .trace_writer import NoopTraceWriter, PerfettoTraceWriter
