"""Span tracer with host-thread and device timelines (tunix/perf/trace.py:87-476).

    with tracer.span_group("global_step"):
      with tracer.span("rollout", devices) as span:
        out = engine.generate(...)
        span.device_end([out])         # device work that the span covers

A thread span ends when its `with` block exits. A device span begins at
`max(thread begin, end of the previous span on that device)` and ends when the work enqueued so
far on the current CUDA stream has completed: `device_end` records a CUDA event and a waiter
thread resolves the end time when the event fires, so tracing never blocks the training thread.
Without a GPU the device span ends at `device_end` time.
"""
from __future__ import annotations

import contextlib
import threading
import time
from typing import Any, Callable, Dict, List, Optional, Sequence

from .span import Span, SpanGroup, span_group_print

MetricsT = Dict[str, Any]


def create_thread_timeline_id() -> str:
  return f"thread-{threading.get_ident()}"


def create_device_timeline_id(id: Any) -> str:
  return id if isinstance(id, str) else f"device-{id}"


def create_device_timeline_ids(devices: Optional[Sequence[Any]]) -> List[str]:
  return [create_device_timeline_id(d) for d in (devices or [])]


class _NoopSpan:

  def device_end(self, waitlist: Any = None) -> None:
    pass

  def async_end(self, waitlist: Any = None) -> None:
    pass


class NoopTracer:
  """Does nothing; the default when perf metrics are not configured."""

  def synchronize(self) -> None:
    pass

  def print(self) -> None:
    pass

  def export(self) -> MetricsT:
    return {}

  @property
  def all_devices(self) -> List[Any]:
    return []

  @contextlib.contextmanager
  def span_group(self, name: str, *a, **k):
    yield

  @contextlib.contextmanager
  def span(self, name: str, devices: Any = None, tags: Any = None, **k):
    yield _NoopSpan()


class Timeline:
  """A tree of span groups plus a stack of the currently open groups."""

  def __init__(self, id: str, born: float):
    self.id = id
    self.born = born
    self.root = SpanGroup("root")
    self.root.begin = born
    self._stack: List[SpanGroup] = [self.root]
    self._last_span: Optional[Span] = None
    self._open_span: Optional[Span] = None
    self._lock = threading.Lock()

  def span_group_begin(self, name: str, begin: float) -> SpanGroup:
    with self._lock:
      g = SpanGroup(name, self._stack[-1])
      g.begin = begin
      self._stack.append(g)
      return g

  def span_group_end(self, end: float) -> None:
    with self._lock:
      if len(self._stack) <= 1:
        raise ValueError(f"{self.id}: no span group is active")
      self._stack.pop().end = end

  def thread_span_begin(self, name: str, begin: float) -> Span:
    with self._lock:
      s = Span(name, begin)
      self._stack[-1].inner.append(s)
      self._open_span = s
      return s

  def thread_span_end(self, end: float) -> None:
    with self._lock:
      if self._open_span is not None:
        self._open_span.end = end
        self._last_span = self._open_span
        self._open_span = None

  def device_span(self, name: str, thread_begin: float) -> Span:
    with self._lock:
      begin = thread_begin
      if self._last_span is not None and self._last_span.ended:
        begin = max(begin, self._last_span.end)
      s = Span(name, begin)
      self._stack[-1].inner.append(s)
      self._last_span = s
      return s


class ThreadTimeline(Timeline):
  pass


class DeviceTimeline(Timeline):

  def __init__(self, id: str, born: float):
    super().__init__(id, born)
    self._pending: List[threading.Thread] = []

  def wait_pending_spans(self) -> None:
    for t in list(self._pending):
      t.join()
    self._pending.clear()


class _ActiveSpan:

  def __init__(self, tracer: "PerfTracer", name: str, thread_begin: float, devices: List[str]):
    self._tracer, self._name, self._begin, self._devices = tracer, name, thread_begin, devices
    self._ended = False

  def device_end(self, waitlist: Any = None) -> None:
    """Declares that the device work of this span is whatever has been enqueued so far."""
    if self._ended or not self._devices:
      return
    self._ended = True
    spans = [self._tracer._get_or_create_device_timeline(d).device_span(self._name, self._begin)
             for d in self._devices]
    ev = None
    try:
      import torch
      if torch.cuda.is_available():
        ev = torch.cuda.Event()
        ev.record()
    except Exception:
      ev = None
    if ev is None:
      now = time.perf_counter()
      for s in spans:
        s.end = now
      return

    def wait():
      ev.synchronize()
      now = time.perf_counter()
      for s in spans:
        s.end = max(now, s.begin)
    t = threading.Thread(target=wait, daemon=True)
    t.start()
    for d in self._devices:
      self._tracer._get_or_create_device_timeline(d)._pending.append(t)

  async_end = device_end


class PerfTracer(NoopTracer):
  """Collects span trees per host thread and per device and hands them to an export function."""

  def __init__(self, devices: Optional[Sequence[Any]] = None,
               export_fn: Optional[Callable[["Any"], MetricsT]] = None):
    self._born = time.perf_counter()
    self._export_fn = export_fn
    self._main_thread_id = create_thread_timeline_id()
    self._thread_timelines: Dict[str, ThreadTimeline] = {}
    self._device_timelines: Dict[str, DeviceTimeline] = {}
    self._lock = threading.Lock()
    self._devices = create_device_timeline_ids(devices)
    for d in self._devices:
      self._get_or_create_device_timeline(d)
    self._get_or_create_thread_timeline(self._main_thread_id)

  def _get_timelines(self) -> Dict[str, Timeline]:
    out: Dict[str, Timeline] = {}
    out.update(self._thread_timelines)
    out.update(self._device_timelines)
    return out

  def _get_or_create_thread_timeline(self, id: str) -> ThreadTimeline:
    with self._lock:
      if id not in self._thread_timelines:
        self._thread_timelines[id] = ThreadTimeline(id, self._born)
      return self._thread_timelines[id]

  def _get_or_create_device_timeline(self, id: str) -> DeviceTimeline:
    with self._lock:
      if id not in self._device_timelines:
        self._device_timelines[id] = DeviceTimeline(id, self._born)
      return self._device_timelines[id]

  def synchronize(self) -> None:
    for t in self._device_timelines.values():
      t.wait_pending_spans()

  def print(self) -> None:
    self.synchronize()
    for t in self._get_timelines().values():
      print(f"== {t.id}")
      span_group_print(t.root, self._born)

  def export(self) -> MetricsT:
    """Runs the export function over everything recorded since the last export, then clears it."""
    if self._export_fn is None:
      return {}
    self.synchronize()
    from .metrics import PerfSpanQuery
    try:
      return self._export_fn(PerfSpanQuery(self._get_timelines(), self._main_thread_id))
    finally:
      for t in self._get_timelines().values():
        with t._lock:
          t.root.inner = [x for x in t.root.inner if isinstance(x, SpanGroup) and x in t._stack]

  @property
  def all_devices(self) -> List[Any]:
    return list(self._devices)

  @contextlib.contextmanager
  def span_group(self, name: str, *a, **k):
    tl = self._get_or_create_thread_timeline(create_thread_timeline_id())
    tl.span_group_begin(name, time.perf_counter())
    try:
      yield
    finally:
      tl.span_group_end(time.perf_counter())

  @contextlib.contextmanager
  def span(self, name: str, devices: Any = None, tags: Any = None, **k):
    begin = time.perf_counter()
    tl = self._get_or_create_thread_timeline(create_thread_timeline_id())
    tl.thread_span_begin(name, begin)
    dev_ids = create_device_timeline_ids(devices) if devices is not None else []
    active = _ActiveSpan(self, name, begin, dev_ids)
    try:
      yield active
    finally:
      tl.thread_span_end(time.perf_counter())
      if dev_ids and not active._ended:
        active.device_end()
