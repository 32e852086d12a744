"""Trace writer: dumps span trees as Chrome trace-event JSON, which the Perfetto UI opens
directly (the reference writes Perfetto protobuf packets, tunix/perf/perfetto.py:36-230; the
event model - one track per timeline, nested complete events - is the same)."""
from __future__ import annotations

import json
import os
import threading
import time
from typing import Any, Dict, List, Optional, Sequence

from .span import Span, SpanGroup


class PerfettoTraceWriter:

  def __init__(self, trace_dir: str = "", file_prefix: str = "perf_trace"):
    self._dir = trace_dir or os.path.join(os.getcwd(), "perf_traces")
    os.makedirs(self._dir, exist_ok=True)
    self._path = os.path.join(self._dir, f"{file_prefix}_{int(time.time())}_{os.getpid()}.json")
    self._events: List[Dict[str, Any]] = []
    self._lock = threading.Lock()
    self._tracks: Dict[str, int] = {}

  def _tid(self, track: str) -> int:
    if track not in self._tracks:
      self._tracks[track] = len(self._tracks) + 1
      self._events.append({"ph": "M", "name": "thread_name", "pid": 1, "tid": self._tracks[track],
                           "args": {"name": track}})
    return self._tracks[track]

  def _add(self, track: str, node, depth: int = 0) -> None:
    if node.end == float("inf"):
      return
    self._events.append({"ph": "X", "name": node.name, "pid": 1, "tid": self._tid(track),
                         "ts": node.begin * 1e6, "dur": max(0.0, (node.end - node.begin) * 1e6)})
    if isinstance(node, SpanGroup):
      for x in node.inner:
        self._add(track, x, depth + 1)

  def log_trace(self, global_step_groups: Sequence[SpanGroup], rollout_spans: Sequence[Span] = (),
                refer_inference_spans: Sequence[Span] = (), actor_train_groups: Sequence[SpanGroup] = ()) -> None:
    with self._lock:
      for g in global_step_groups:
        self._add("main", g)
      for s in rollout_spans:
        self._add("rollout", s)
      for s in refer_inference_spans:
        self._add("reference", s)
      for g in actor_train_groups:
        self._add("actor", g)
      self.flush()

  def log_timelines(self, timelines: Dict[str, Any]) -> None:
    with self._lock:
      for tid, tl in timelines.items():
        for x in tl.root.inner:
          self._add(tid, x)
      self.flush()

  def flush(self) -> None:
    tmp = self._path + ".tmp"
    with open(tmp, "w") as f:
      json.dump({"traceEvents": self._events, "displayTimeUnit": "ms"}, f)
    os.replace(tmp, self._path)

  @property
  def path(self) -> str:
    return self._path
