"""Export side of the tag-based tracer (tunix/perf/experimental/export.py:34-160).

`PerfMetricsExport.export_metrics` is the export function a `PerfTracer` is given. It never writes on the
training thread: timelines go onto a single-consumer queue and a daemon writer thread drains it in order into the
trace writer. Writing is best effort - a failed write is logged and the next one is still tried; after `shutdown`
later exports are dropped with a warning. The device-to-role table that names the trace's tracks comes from a
cluster config's role meshes (`from_cluster_config`).
"""
from __future__ import annotations

import logging
import queue
import threading
from typing import Any, Dict, List, Mapping, Optional

from . import trace_writer as trace_writer_lib
from .timeline import Timeline

log = logging.getLogger(__name__)
MetricsT = Dict[str, Any]
DEFAULT_TRACE_DIR = "/tmp/perf_traces"
_STOP = object()


def log_metric_export_fn(timelines: Mapping[str, Timeline]) -> MetricsT:
  log.info("\n=== Exporting Timelines ===\n %s", timelines)
  return {}


def _devices_of_mesh(mesh: Any) -> List[int]:
  if mesh is None:
    return [0]
  if hasattr(mesh, "ranks"):
    return list(mesh.ranks())
  return list(getattr(mesh, "devices").flatten().tolist())


class _WriterThread:
  """Feeds timelines to a trace writer, one at a time, off the caller's thread."""

  def __init__(self, writer: trace_writer_lib.TraceWriter):
    self._writer = writer
    self._inbox: "queue.Queue[Any]" = queue.Queue()
    self._thread = threading.Thread(target=self._drain, daemon=True, name="PerfExport")
    self._thread.start()
    self.open = True

  def _drain(self) -> None:
    while True:
      item = self._inbox.get()
      if item is _STOP:
        return
      try:
        self._writer.write_timelines(item)
      except Exception:  # noqa: BLE001 - tracing must not take training down
        log.exception("Background trace export failed.")

  def put(self, timelines: Mapping[str, Timeline]) -> None:
    self._inbox.put(timelines)

  def stop(self, wait: bool) -> None:
    if not self.open:
      return
    self.open = False
    self._inbox.put(_STOP)
    if wait:
      self._thread.join()


class PerfMetricsExport:

  def __init__(self, *, enable_trace_writer: bool = True, trace_dir: Optional[str] = None,
               role_to_devices: Optional[Mapping[str, Any]] = None):
    self._trace_writer_enabled = enable_trace_writer
    if enable_trace_writer:
      self._writer: trace_writer_lib.TraceWriter = trace_writer_lib.PerfettoTraceWriter(
          trace_dir or DEFAULT_TRACE_DIR, role_to_devices=role_to_devices)
      self._background: Optional[_WriterThread] = _WriterThread(self._writer)
    else:
      self._writer = trace_writer_lib.NoopTraceWriter()
      self._background = None

  @classmethod
  def from_cluster_config(cls, cluster_config: Any, enable_trace_writer: bool = True,
                          trace_dir: Optional[str] = None) -> "PerfMetricsExport":
    meshes = getattr(cluster_config, "role_to_mesh", None) or {}
    table = {getattr(role, "value", str(role)): _devices_of_mesh(mesh) for role, mesh in meshes.items()}
    return cls(enable_trace_writer=enable_trace_writer, trace_dir=trace_dir, role_to_devices=table)

  @property
  def writer(self) -> trace_writer_lib.TraceWriter:
    return self._writer

  def export_metrics(self, timelines: Mapping[str, Timeline]) -> MetricsT:
    if not self._trace_writer_enabled:
      return {}
    if self._background is None or not self._background.open:
      log.warning("PerfMetricsExport background worker has been shut down. Cannot write metrics.")
      return {}
    self._background.put(timelines)
    return {}

  def shutdown(self, wait: bool = True) -> None:
    if self._background is not None:
      self._background.stop(wait)
      self._background = None

  def __enter__(self) -> "PerfMetricsExport":
    return self

  def __exit__(self, exc_type, exc, tb) -> None:
    self.shutdown()
