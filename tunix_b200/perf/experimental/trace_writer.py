"""Writes timelines as a Chrome/Perfetto JSON trace (loads in ui.perfetto.dev).

Each call appends the steps committed since the previous call. One process track per group
("host", one per role with its devices, "queue"), one thread track per timeline and lane:
spans of a timeline that overlap in time (asynchronous device spans) are spread over lanes so
none hides another. Span names carry their identifying tags (step, micro-batch, group id).

Counterpart of tunix/perf/experimental/trace_writer.py:42-389, with the JSON trace-event format
instead of the protobuf one.
"""
from __future__ import annotations

import abc
import json
import logging
import os
import threading
import time
from typing import Any, Dict, List, Mapping, Optional, Sequence, Tuple

from . import constants
from . import timeline_utils
from .timeline import Span, Timeline

log = logging.getLogger(__name__)
_NAME_TAGS = (constants.STEP, constants.MINI_BATCH, constants.MICRO_BATCH, constants.GROUP_ID, constants.PAIR_INDEX)


def _create_span_name(name: str, tags: Mapping[str, Any]) -> str:
  """"rollout [step=3, group_id=7]"; a NAME tag replaces the base name."""
  base = str(tags.get(constants.NAME, name)) if tags else name
  parts = [f"{k}={tags[k]}" for k in _NAME_TAGS if tags and k in tags]
  return f"{base} [{', '.join(parts)}]" if parts else base


def _assign_lanes(spans: Sequence[Span]) -> List[Tuple[Span, int]]:
  """Greedy interval colouring in begin order; children may share their parent's lane."""
  lanes_end: List[float] = []
  out = []
  for sp in sorted(spans, key=lambda s: (s.begin, -s.end)):
    for i, end in enumerate(lanes_end):
      if sp.begin >= end:
        lanes_end[i] = sp.end
        out.append((sp, i))
        break
    else:
      lanes_end.append(sp.end)
      out.append((sp, len(lanes_end) - 1))
  return out


class TraceWriter(abc.ABC):

  @abc.abstractmethod
  def write_timelines(self, timelines: Mapping[str, Timeline]) -> None:
    ...


class NoopTraceWriter(TraceWriter):

  def write_timelines(self, timelines: Mapping[str, Timeline]) -> None:
    del timelines


class PerfettoTraceWriter(TraceWriter):

  def __init__(self, trace_dir: str, role_to_devices: Optional[Mapping[str, Any]] = None):
    self._trace_dir = trace_dir
    self._role_to_devices = {str(r): timeline_utils.generate_device_timeline_ids(list(d))
                             for r, d in (role_to_devices or {}).items()}
    self._written_steps: Dict[str, int] = {}
    self._pids: Dict[str, int] = {}
    self._tids: Dict[Tuple[str, int], int] = {}
    self._events: List[dict] = []
    self._lock = threading.Lock()
    self._path = None
    try:
      os.makedirs(trace_dir, exist_ok=True)
      self._path = os.path.join(trace_dir, f"perfetto_trace_v2_{int(time.time())}_{os.getpid()}.json")
    except OSError:
      log.exception("cannot create trace directory %s; tracing disabled", trace_dir)

  @property
  def path(self) -> Optional[str]:
    return self._path

  def _get_device_track_name(self, tl_id: str) -> Optional[str]:
    base = tl_id[:-len("_queue")] if timeline_utils.is_queued_timeline(tl_id) else tl_id
    roles = [r for r, devs in self._role_to_devices.items() if base in devs]
    return "/".join(sorted(roles)) if roles else None

  def _track(self, tl_id: str) -> str:
    if timeline_utils.is_host_timeline(tl_id):
      return "host"
    name = self._get_device_track_name(tl_id) or "devices"
    return f"{name} (queued)" if timeline_utils.is_queued_timeline(tl_id) else name

  def _ids(self, tl_id: str, lane: int) -> Tuple[int, int]:
    track = self._track(tl_id)
    if track not in self._pids:
      self._pids[track] = len(self._pids) + 1
      self._events.append({"ph": "M", "name": "process_name", "pid": self._pids[track], "args": {"name": track}})
    key = (tl_id, lane)
    if key not in self._tids:
      self._tids[key] = len(self._tids) + 1
      label = tl_id if lane == 0 else f"{tl_id} #{lane}"
      self._events.append({"ph": "M", "name": "thread_name", "pid": self._pids[track], "tid": self._tids[key],
                           "args": {"name": label}})
    return self._pids[track], self._tids[key]

  def write_timelines(self, timelines: Mapping[str, Timeline]) -> None:
    if self._path is None:
      return
    with self._lock:
      for tl_id, tl in timelines.items():
        steps = tl.committed_steps
        first = self._written_steps.get(tl_id, 0)
        for step in steps[first:]:
          for sp, lane in _assign_lanes([s for s in step.values() if s.ended]):
            pid, tid = self._ids(tl_id, lane)
            self._events.append({
                "ph": "X", "name": _create_span_name(sp.name, sp.tags or {}), "pid": pid, "tid": tid,
                "ts": (sp.begin - tl.born) * 1e6, "dur": max(sp.duration, 0.0) * 1e6,
                "args": {k: (v if isinstance(v, (int, float, str, bool)) else str(v))
                         for k, v in (sp.tags or {}).items()}})
        self._written_steps[tl_id] = len(steps)
      tmp = self._path + ".tmp"
      with open(tmp, "w", encoding="utf-8") as f:
        json.dump({"traceEvents": self._events, "displayTimeUnit": "ms"}, f)
      os.replace(tmp, self._path)
