"""Performance tracing: span trees per host thread / device, metric export, trace files."""
from .export import PerfMetricsExport  # noqa: F401
from .metrics import PerfMetricsConfig, PerfMetricsOptions, PerfSpanQuery  # noqa: F401
from .trace import NoopTracer, PerfTracer  # noqa: F401
