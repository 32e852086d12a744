"""Export functions for the tag-based tracer (tunix/perf/experimental/export.py:34-160)."""
from __future__ import annotations

import concurrent.futures
import logging
from typing import Any, Dict, Mapping, Optional

from . import trace_writer as trace_writer_lib
from .timeline import Timeline

log = logging.getLogger(__name__)
MetricsT = Dict[str, Any]
DEFAULT_TRACE_DIR = "/tmp/perf_traces"


def log_metric_export_fn(timelines: Mapping[str, Timeline]) -> MetricsT:
  log.info("\n=== Exporting Timelines ===\n %s", timelines)
  return {}


class PerfMetricsExport:
  """Hands committed timelines to a trace writer on a background thread; `export_metrics` is
  the export function to give the tracer. Writing is best effort: errors are logged."""

  @classmethod
  def from_cluster_config(cls, cluster_config: Any, enable_trace_writer: bool = True,
                          trace_dir: Optional[str] = None) -> "PerfMetricsExport":
    role_to_devices = {}
    for role, mesh in (getattr(cluster_config, "role_to_mesh", None) or {}).items():
      name = role.value if hasattr(role, "value") else str(role)
      if mesh is None:
        role_to_devices[name] = [0]
      elif hasattr(mesh, "ranks"):
        role_to_devices[name] = list(mesh.ranks())
      else:
        role_to_devices[name] = list(getattr(mesh, "devices").flatten().tolist())
    return cls(enable_trace_writer=enable_trace_writer, trace_dir=trace_dir, role_to_devices=role_to_devices)

  def __init__(self, *, enable_trace_writer: bool = True, trace_dir: Optional[str] = None,
               role_to_devices: Optional[Mapping[str, Any]] = None):
    self._trace_writer_enabled = enable_trace_writer
    if enable_trace_writer:
      self._writer: trace_writer_lib.TraceWriter = trace_writer_lib.PerfettoTraceWriter(
          trace_dir or DEFAULT_TRACE_DIR, role_to_devices=role_to_devices)
      self._executor: Optional[concurrent.futures.ThreadPoolExecutor] = concurrent.futures.ThreadPoolExecutor(
          max_workers=1, thread_name_prefix="PerfExport")
    else:
      self._writer = trace_writer_lib.NoopTraceWriter()
      self._executor = None

  @property
  def writer(self) -> trace_writer_lib.TraceWriter:
    return self._writer

  def _safe_write(self, timelines: Mapping[str, Timeline]) -> None:
    try:
      self._writer.write_timelines(timelines)
    except Exception:  # pylint: disable=broad-exception-caught
      log.exception("Background trace export failed.")

  def export_metrics(self, timelines: Mapping[str, Timeline]) -> MetricsT:
    if self._trace_writer_enabled:
      if self._executor is not None:
        self._executor.submit(self._safe_write, timelines)
      else:
        log.warning("PerfMetricsExport background worker has been shut down. Cannot write metrics.")
    return {}

  def shutdown(self, wait: bool = True) -> None:
    if self._executor is not None:
      self._executor.shutdown(wait=wait)
      self._executor = None

  def __enter__(self) -> "PerfMetricsExport":
    return self

  def __exit__(self, exc_type, exc, tb) -> None:
    self.shutdown()
