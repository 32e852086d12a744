"""Perf metric options and the span query DSL (tunix/perf/metrics.py:66-227)."""
from __future__ import annotations

import dataclasses
import logging
from typing import Any, Callable, Dict, List, Mapping, Optional, Tuple

from .span import (SpanGroup, span_group_batch_query_all, span_group_batch_query_first,
                   span_group_batch_query_last, span_group_batch_query_nth)

log = logging.getLogger(__name__)
MetricsT = Dict[str, Tuple[Any, Optional[Callable]]]


@dataclasses.dataclass
class MetricsBuffer:
  global_steps: int
  metrics: Dict[str, Tuple[List[Any], Optional[Callable]]] = dataclasses.field(default_factory=dict)
  mode: str = "train"


@dataclasses.dataclass(frozen=True)
class PerfMetricsOptions:
  enable_perf_v1: bool = True
  enable_perf_v2: bool = False
  custom_export_fn_path: str = ""
  custom_export_fn_path_v2: str = ""
  enable_trace_writer: bool = True
  trace_dir: str = ""

  def __post_init__(self):
    if self.custom_export_fn_path and not self.enable_perf_v1:
      raise ValueError("custom_export_fn_path is set but enable_perf_v1 is False.")
    if self.custom_export_fn_path_v2 and not self.enable_perf_v2:
      raise ValueError("custom_export_fn_path_v2 is set but enable_perf_v2 is False.")
    if self.enable_trace_writer and not (self.enable_perf_v1 or self.enable_perf_v2):
      raise ValueError("enable_trace_writer is True but neither perf v1 nor v2 is enabled.")
    if self.trace_dir and not self.enable_trace_writer:
      log.warning("trace_dir is set to %r but enable_trace_writer is False.", self.trace_dir)


@dataclasses.dataclass
class PerfMetricsConfig:
  custom_export_fn: Optional[Callable[["PerfSpanQuery"], MetricsT]] = None
  custom_export_fn_v2: Optional[Callable[[Mapping[str, Any]], MetricsT]] = None


class PerfSpanQuery:
  """Chainable query over timelines:

      query().main().last_group("global_step").all_groups("mini_batch_step").get()
      query().timeline("device-0").last_group("global_step").get()
  """

  def __init__(self, timelines: Mapping[str, Any], main_thread_id: str):
    self._timelines = timelines
    self._main_thread_id = main_thread_id
    self._select: List[SpanGroup] = []

  def __call__(self) -> "PerfSpanQuery":
    return PerfSpanQuery(self._timelines, self._main_thread_id)

  def get_main_thread_id(self) -> str:
    return self._main_thread_id

  def get_timeline_ids(self) -> List[str]:
    return list(self._timelines.keys())

  def timeline(self, id: str) -> "PerfSpanQuery":
    self._select = [self._timelines[id].root] if id in self._timelines else []
    return self

  def main(self) -> "PerfSpanQuery":
    return self.timeline(self._main_thread_id)

  def first_group(self, name: str) -> "PerfSpanQuery":
    self._select = span_group_batch_query_first(self._select, name)
    return self

  def last_group(self, name: str) -> "PerfSpanQuery":
    self._select = span_group_batch_query_last(self._select, name)
    return self

  def nth_group(self, name: str, index: int) -> "PerfSpanQuery":
    self._select = span_group_batch_query_nth(self._select, name, index)
    return self

  def all_groups(self, name: str) -> "PerfSpanQuery":
    self._select = span_group_batch_query_all(self._select, name)
    return self

  def get(self) -> List[SpanGroup]:
    return self._select
