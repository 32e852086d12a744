"""OpenTelemetry metric exporter that forwards gauge points to a Weights & Biases run
(tunix/sft/otel_wandb.py:98-157). Both packages are optional; importing this module without
them works, constructing the exporter does not."""
from __future__ import annotations

from typing import Any, Optional

try:
  from opentelemetry.sdk.metrics.export import MetricExporter, MetricExportResult
except Exception:  # pragma: no cover
  MetricExporter = object
  MetricExportResult = None


class WandbMetricsExporter(MetricExporter):  # type: ignore[misc]

  def __init__(self, run: Any = None, **init_kwargs):
    if MetricExportResult is None:
      raise ImportError("opentelemetry-sdk is required for WandbMetricsExporter")
    super().__init__()
    if run is None:
      import wandb
      run = wandb.init(**init_kwargs)
    self._run = run

  def export(self, metrics_data, timeout_millis: float = 10_000, **kwargs):
    try:
      for rm in metrics_data.resource_metrics:
        for sm in rm.scope_metrics:
          for metric in sm.metrics:
            for pt in metric.data.data_points:
              attrs = dict(pt.attributes or {})
              prefix = attrs.get("tunix.metrics_prefix", "")
              mode = attrs.get("tunix.mode", "")
              key = "/".join(x for x in (prefix, mode, metric.name) if x)
              self._run.log({key: pt.value})
      return MetricExportResult.SUCCESS
    except Exception:
      return MetricExportResult.FAILURE

  def force_flush(self, timeout_millis: float = 10_000) -> bool:
    return True

  def shutdown(self, timeout_millis: float = 30_000, **kwargs) -> None:
    try:
      self._run.finish()
    except Exception:
      pass
