"""Metrics logger with pluggable backends.

Keeps a local history `{prefix: {mode: {name: [values]}}}` and fans every scalar out, under the
event name `"{prefix}/{mode}/{name}"`, to the live backends on rank 0: a JSON-lines file (always
available), TensorBoard and Weights & Biases when their packages import, user factories under
`backend_kwargs["custom_backend"]`, and optionally an OpenTelemetry gauge (double write).
Mirrors tunix/sft/metrics_logger.py:121-399.
"""
from __future__ import annotations

import collections
import dataclasses
import enum
import json
import logging
import os
import re
import threading
import time
from typing import Any, Callable, Dict, List, Optional, Protocol, Union

import numpy as np

log = logging.getLogger(__name__)

try:  # optional
  from opentelemetry import metrics as otel_metrics
except Exception:  # pragma: no cover
  otel_metrics = None


def _process_index() -> int:
  return int(os.environ.get("RANK", "0"))


class LoggingBackend(Protocol):

  def log_scalar(self, event: str, value: Any, **kwargs) -> None:
    ...

  def close(self) -> None:
    ...


def _scalar(v: Any) -> float:
  try:
    import torch
    if isinstance(v, torch.Tensor):
      return float(v.detach().float().mean().item())
  except Exception:
    pass
  return float(np.asarray(v, dtype=np.float64).mean())


class JsonlBackend:
  """Appends `{"event", "value", "step", "time"}` lines to `<log_dir>/metrics.jsonl`."""

  def __init__(self, log_dir: str, flush_every_n_steps: int = 100):
    os.makedirs(log_dir, exist_ok=True)
    self._f = open(os.path.join(log_dir, "metrics.jsonl"), "a")
    self._n = 0
    self._every = max(1, flush_every_n_steps)
    self._lock = threading.Lock()

  def log_scalar(self, event: str, value: Any, **kwargs) -> None:
    with self._lock:
      self._f.write(json.dumps({"event": event, "value": _scalar(value), "step": kwargs.get("step"),
                                "time": time.time()}) + "\n")
      self._n += 1
      if self._n % self._every == 0:
        self._f.flush()

  def close(self) -> None:
    with self._lock:
      if not self._f.closed:
        self._f.flush()
        self._f.close()


class TensorboardBackend:

  def __init__(self, log_dir: str, flush_every_n_steps: int = 100, **kwargs):
    from torch.utils.tensorboard import SummaryWriter  # raises ImportError when tensorboard is absent
    self._w = SummaryWriter(log_dir=log_dir, **kwargs)
    self._n = 0
    self._every = max(1, flush_every_n_steps)

  def log_scalar(self, event: str, value: Any, **kwargs) -> None:
    self._w.add_scalar(event, _scalar(value), global_step=kwargs.get("step"))
    self._n += 1
    if self._n % self._every == 0:
      self._w.flush()

  def close(self) -> None:
    self._w.close()


class WandbBackend:

  def __init__(self, project: str, name: str = "", **kwargs):
    import wandb  # raises ImportError when absent
    self._wandb = wandb
    self._run = wandb.init(project=project, name=name or None, **kwargs)

  def log_scalar(self, event: str, value: Any, **kwargs) -> None:
    self._wandb.log({event: _scalar(value)}, step=kwargs.get("step"))

  def close(self) -> None:
    self._wandb.finish()


BackendFactory = Callable[[], LoggingBackend]


@dataclasses.dataclass
class MetricsLoggerOptions:
  """Where and how metrics are written."""

  log_dir: str
  project_name: str = "tunix"
  run_name: str = ""
  flush_every_n_steps: int = 100
  # {'wandb': {...}, 'tensorboard': {...}, 'jsonl': {...}} keyword arguments per backend, or
  # {'custom_backend': [factory, ...]} to replace the defaults.
  backend_kwargs: Dict[str, Any] = dataclasses.field(default_factory=dict)
  enable_opentelemetry: bool = False

  def create_backends(self) -> List[LoggingBackend]:
    if _process_index() != 0:
      return []
    kw = self.backend_kwargs or {}
    if kw.get("custom_backend"):
      return [factory() for factory in kw["custom_backend"]]
    backends: List[LoggingBackend] = [JsonlBackend(self.log_dir, self.flush_every_n_steps, **kw.get("jsonl", {}))]
    try:
      backends.append(TensorboardBackend(log_dir=self.log_dir, flush_every_n_steps=self.flush_every_n_steps,
                                         **kw.get("tensorboard", {})))
    except Exception as e:  # tensorboard not installed
      log.info("TensorboardBackend skipped: %s", e)
    if "wandb" in kw or os.environ.get("WANDB_API_KEY") or os.environ.get("WANDB_MODE"):
      try:
        backends.append(WandbBackend(project=self.project_name, name=self.run_name, **kw.get("wandb", {})))
      except Exception as e:
        log.info("WandbBackend skipped: %s", e)
    return backends


class Mode(str, enum.Enum):
  TRAIN = "train"
  EVAL = "eval"

  def __str__(self):
    return self.value


def _calculate_geometric_mean(x: np.ndarray) -> np.ndarray:
  return np.exp(np.mean(np.log(x)))


_OTEL_NAME = re.compile(r"[^a-zA-Z0-9_.-]+")
_OTEL_KNOWN = {
    "loss": "tunix.training.loss",
    "perplexity": "tunix.training.perplexity",
    "learning_rate": "tunix.training.learning_rate",
    "grad_norm": "tunix.training.gradient.norm",
}


def _otel_name(metric_name: str) -> str:
  if metric_name in _OTEL_KNOWN:
    return _OTEL_KNOWN[metric_name]
  n = _OTEL_NAME.sub(".", metric_name).strip(".") or "unnamed"
  return f"tunix.{n.lower()}"


class MetricsLogger:
  """Logs scalars to the local history and to every live backend."""

  def __init__(self, metrics_logger_options: Optional[MetricsLoggerOptions] = None, *,
               otel_meter_provider: Any = None):
    self._metrics: Dict[str, Dict[Any, Dict[str, list]]] = {}
    self._backends = metrics_logger_options.create_backends() if metrics_logger_options else []
    self._otel_meter = None
    self._otel_gauges: Dict[str, Any] = {}
    self._otel_lock = threading.Lock()
    if metrics_logger_options and metrics_logger_options.enable_opentelemetry:
      if otel_metrics is None and otel_meter_provider is None:
        raise ImportError("MetricsLoggerOptions.enable_opentelemetry is set but the OpenTelemetry API is not "
                          "installed.")
      provider = otel_meter_provider or otel_metrics.get_meter_provider()
      self._otel_meter = provider.get_meter("tunix")

  def log(self, metrics_prefix: str, metric_name: str, scalar_value: Any, mode: Union[Mode, str], step: int):
    mode_key = str(mode)
    hist = self._metrics.setdefault(metrics_prefix, {}).setdefault(mode_key, collections.defaultdict(list))
    value = np.asarray(_scalar(scalar_value), dtype=np.float64)
    hist[metric_name].append(value)
    event = f"{metrics_prefix}/{mode_key}/{metric_name}"
    for b in self._backends:
      try:
        b.log_scalar(event, value, step=step)
      except Exception:  # a failing backend must not interrupt training
        log.exception("metrics backend %r failed for %s", type(b).__name__, event)
    if self._otel_meter is not None:
      try:
        self._emit_otel(metrics_prefix, metric_name, float(value), mode_key, step)
      except Exception:
        log.exception("Failed to emit OpenTelemetry metric %s", event)

  def _emit_otel(self, prefix: str, name: str, value: float, mode: str, step: int) -> None:
    oname = _otel_name(name)
    with self._otel_lock:
      g = self._otel_gauges.get(oname)
      if g is None:
        g = self._otel_meter.create_gauge(oname, unit="1", description=f"Tunix metric {name!r}")
        self._otel_gauges[oname] = g
      sg = self._otel_gauges.get("tunix.training.step")
      if sg is None:
        sg = self._otel_meter.create_gauge("tunix.training.step", unit="{step}", description="logical step")
        self._otel_gauges["tunix.training.step"] = sg
    attrs = {"tunix.metrics_prefix": prefix, "tunix.mode": mode}
    g.set(value, attrs)
    if step is not None:
      sg.set(step, attrs)

  def metric_exists(self, metrics_prefix, metric_name: str, mode: Union[Mode, str]) -> bool:
    mode = str(mode)
    return (metrics_prefix in self._metrics and mode in self._metrics[metrics_prefix]
            and metric_name in self._metrics[metrics_prefix][mode])

  def get_metric(self, metrics_prefix, metric_name: str, mode: Union[Mode, str]):
    """Mean of the logged values (geometric mean for perplexity)."""
    if not self.metric_exists(metrics_prefix, metric_name, mode):
      raise ValueError(f"Metric '{metrics_prefix}/{mode}/{metric_name}' not found.")
    values = np.stack(self._metrics[metrics_prefix][str(mode)][metric_name])
    if metric_name == "perplexity":
      return _calculate_geometric_mean(values)
    return np.mean(values)

  def get_metric_history(self, metrics_prefix, metric_name: str, mode: Union[Mode, str]):
    if not self.metric_exists(metrics_prefix, metric_name, mode):
      avail = list(self._metrics.get(metrics_prefix, {}).get(str(mode), {}).keys())
      raise ValueError(f" Metric '{metrics_prefix}/{mode}/{metric_name}' not found. Available metrics for mode "
                       f"'{mode}': {avail}")
    return np.stack(self._metrics[metrics_prefix][str(mode)][metric_name])

  def close(self):
    for b in self._backends:
      try:
        b.close()
      except Exception:
        log.exception("closing metrics backend failed")
    self._backends = []
