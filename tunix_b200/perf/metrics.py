"""Perf metric options and the span query DSL (tunix/perf/metrics.py:66-227)."""
from __future__ import annotations

import dataclasses
import logging
from typing import Any, Callable, Dict, List, Mapping, Optional, Tuple

from .span import SpanGroup

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
    # (the option that is set, what it needs, is the combination fatal)
    needs = (("custom_export_fn_path", self.enable_perf_v1, "enable_perf_v1 is False", True),
             ("custom_export_fn_path_v2", self.enable_perf_v2, "enable_perf_v2 is False", True),
             ("enable_trace_writer", self.enable_perf_v1 or self.enable_perf_v2,
              "neither perf v1 nor v2 is enabled", True),
             ("trace_dir", self.enable_trace_writer, "enable_trace_writer is False", False))
    for option, satisfied, why, fatal in needs:
      value = getattr(self, option)
      if not value or satisfied:
        continue
      message = f"{option} is set to {value!r} but {why}."
      if fatal:
        raise ValueError(message)
      log.warning(message)


@dataclasses.dataclass
class PerfMetricsConfig:
  custom_export_fn: Optional[Callable[["PerfSpanQuery"], MetricsT]] = None
  custom_export_fn_v2: Optional[Callable[[Mapping[str, Any]], MetricsT]] = None


class PerfSpanQuery:
  """Chainable query over timelines:

      query().main().last_group("global_step").all_groups("mini_batch_step").get()
      query().timeline("device-0").last_group("global_step").get()

  The selection is a list of groups; every `*_group(s)` step replaces each selected group by some of its direct
  child groups of the given name, chosen by one slice of the matching children (`_descend`). Calling the query
  object starts a fresh query over the same timelines.
  """

  def __init__(self, timelines: Mapping[str, Any], main_thread_id: str):
    self._timelines = timelines
    self._main_thread_id = main_thread_id
    self._select: List[SpanGroup] = []

  def __call__(self) -> "PerfSpanQuery":
    return type(self)(self._timelines, self._main_thread_id)

  def get_main_thread_id(self) -> str:
    return self._main_thread_id

  def get_timeline_ids(self) -> List[str]:
    return [*self._timelines]

  def timeline(self, id: str) -> "PerfSpanQuery":
    found = self._timelines.get(id)
    self._select = [] if found is None else [found.root]
    return self

  def main(self) -> "PerfSpanQuery":
    return self.timeline(self._main_thread_id)

  def _descend(self, name: str, which: slice) -> "PerfSpanQuery":
    self._select = [child for group in self._select for child in group.find_all_inner_groups(name)[which]]
    return self

  def first_group(self, name: str) -> "PerfSpanQuery":
    return self._descend(name, slice(0, 1))

  def last_group(self, name: str) -> "PerfSpanQuery":
    return self._descend(name, slice(-1, None))

  def nth_group(self, name: str, index: int) -> "PerfSpanQuery":
    """Groups with fewer than |index| matching children drop out of the selection."""
    return self._descend(name, slice(index, index + 1) if index >= 0 else _from_end(index))

  def all_groups(self, name: str) -> "PerfSpanQuery":
    return self._descend(name, slice(None))

  def get(self) -> List[SpanGroup]:
    return self._select


def _from_end(index: int) -> slice:
  """The slice selecting exactly element `index` (< 0), empty when the list is shorter than |index|."""
  return slice(index, index + 1) if index != -1 else slice(-1, None)
