"""Tracer front end (tunix/perf/experimental/tracer.py:45-352).

    with tracer.span("rollout", devices=[0, 1], tags={constants.STEP: 3}) as wl:
      out = engine.generate(...)
      wl.async_end(out_event_or_tensor)      # the device lanes close when this is ready

The host span closes when the `with` block exits; each device lane gets a span that begins at
the same host time and ends when the waitlist is ready. `export()` sequentialises overlapping
device spans into active + queued parts (unless the span names are declared concurrent),
commits the step on every timeline and hands the timelines to the export function.
"""
from __future__ import annotations

import collections
import contextlib
import threading
import time
from typing import Any, Callable, Dict, Iterator, List, Mapping, Optional, Sequence, Union

import numpy as np

from . import timeline_utils
from .timeline import AsyncTimeline, BatchAsyncTimelines, Timeline

MetricsT = Dict[str, Any]


def _synchronize_devices() -> None:
  try:
    import torch
    if torch.cuda.is_available():
      torch.cuda.synchronize()
  except ImportError:   # pragma: no cover
    pass


class AsyncWaitlist:

  def __init__(self) -> None:
    self._items: List[Any] = []

  def async_end(self, waitlist: Any) -> None:
    self._items.append(waitlist)

  # the v1 spelling
  device_end = async_end

  @property
  def waitlist(self) -> List[Any]:
    return self._items


class NoopTracer:

  def synchronize(self) -> None:
    pass

  def print(self) -> None:
    pass

  def export(self) -> MetricsT:
    return {}

  @property
  def all_devices(self) -> Sequence[str]:
    return []

  @contextlib.contextmanager
  def span(self, name: str, devices: Any = None, tags: Optional[Mapping[str, Any]] = None) -> Iterator[AsyncWaitlist]:
    yield AsyncWaitlist()


class PerfTracer(NoopTracer):

  def __init__(self, devices: Optional[Sequence[Any]] = None,
               export_fn: Optional[Callable[[Mapping[str, Timeline]], MetricsT]] = None,
               concurrent_spans: Union[None, str, Sequence[str]] = None,
               collect_on_first_device_per_mesh: bool = False):
    """`concurrent_spans`: span names that really overlap on a device (or "all"): timelines that
    contain them are not sequentialised."""
    self._born = time.perf_counter()
    self._export_fn = export_fn
    self._concurrent_spans = concurrent_spans
    self._collect_on_first_device_per_mesh = collect_on_first_device_per_mesh
    self._timelines_lock = threading.RLock()
    self._host_timelines: Dict[str, Timeline] = {}
    self._device_timelines: Dict[str, AsyncTimeline] = {}
    self._device_queue_timelines: Dict[str, Timeline] = collections.defaultdict(self._new_queue_timeline)
    for d in timeline_utils.generate_device_timeline_ids(devices):
      self._get_or_create_device_timeline(d)
    self._get_or_create_host_timeline(timeline_utils.generate_host_timeline_id())

  def _new_queue_timeline(self) -> Timeline:
    return Timeline("queue", self._born)

  def _get_timelines(self) -> Dict[str, Timeline]:
    with self._timelines_lock:
      out: Dict[str, Timeline] = {}
      out.update(self._host_timelines)
      out.update(self._device_timelines)
      out.update(self._device_queue_timelines)
      return out

  def _get_or_create_host_timeline(self, timeline_id: str) -> Timeline:
    with self._timelines_lock:
      if timeline_id not in self._host_timelines:
        self._host_timelines[timeline_id] = Timeline(timeline_id, self._born)
      return self._host_timelines[timeline_id]

  def _get_or_create_device_timeline(self, timeline_id: str) -> AsyncTimeline:
    with self._timelines_lock:
      if timeline_id not in self._device_timelines:
        self._device_timelines[timeline_id] = AsyncTimeline(timeline_id, self._born)
      return self._device_timelines[timeline_id]

  def _get_or_create_device_timelines(self, devices: Any) -> BatchAsyncTimelines:
    return BatchAsyncTimelines([self._get_or_create_device_timeline(i)
                                for i in timeline_utils.generate_device_timeline_ids(devices)])

  def synchronize(self) -> None:
    _synchronize_devices()
    with self._timelines_lock:
      tls = list(self._device_timelines.values())
    for tl in tls:
      tl.wait_pending_spans()

  def print(self) -> None:
    self.synchronize()
    for tl in self._get_timelines().values():
      print(repr(tl))

  def _sequentialize_device_timeline(self, timeline_id: str, tl: AsyncTimeline) -> None:
    with tl._lock:
      ignore = self._concurrent_spans or []
      if any(sp.name in ignore for sp in tl._cur_step.values()):
        return
      active, queued = timeline_utils.sequentialize_overlapping_spans(tl._cur_step)
      tl._cur_step = dict(active)
    if queued:
      qid = timeline_utils.generate_queued_timeline_id(timeline_id)
      qtl = self._device_queue_timelines[qid]
      qtl.id = qid
      with qtl._lock:
        qtl._cur_step.update(queued)

  def process_and_commit_timelines(self) -> None:
    with self._timelines_lock:
      for tl in self._device_timelines.values():
        tl.wait_pending_spans()
      if self._concurrent_spans != "all":
        for tid, tl in list(self._device_timelines.items()):
          self._sequentialize_device_timeline(tid, tl)
      for group in (self._host_timelines, self._device_timelines, self._device_queue_timelines):
        for tl in group.values():
          tl.commit_step()

  def export(self) -> MetricsT:
    if self._export_fn is None:
      return {}
    self.process_and_commit_timelines()
    return self._export_fn(self._get_timelines())

  @property
  def all_devices(self) -> Sequence[str]:
    with self._timelines_lock:
      return list(self._device_timelines.keys())

  @contextlib.contextmanager
  def span(self, name: str, devices: Any = None, tags: Optional[Mapping[str, Any]] = None) -> Iterator[AsyncWaitlist]:
    span_devices = devices
    if self._collect_on_first_device_per_mesh and devices is not None:
      flat = devices.flatten().tolist() if isinstance(devices, np.ndarray) else list(devices)
      span_devices = flat[:1]
    begin = time.perf_counter()
    wl = AsyncWaitlist()
    host_tl = None
    try:
      host_tl = self._get_or_create_host_timeline(timeline_utils.generate_host_timeline_id())
      host_tl.start_span(name, begin, tags=tags)
      yield wl
    finally:
      if host_tl is not None:
        host_tl.stop_span(time.perf_counter())
        self._get_or_create_device_timelines(span_devices).span(name, begin, wl.waitlist, tags=tags)


Tracer = Union[PerfTracer, NoopTracer]
