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


class _Lanes:
  """The tracer's timelines by kind: host threads, device lanes, and the queue lanes that receive the waiting
  part of overlapping device spans. Lanes are created on first use; one lock guards the three tables."""

  def __init__(self, born: float):
    self.born = born
    self.lock = threading.RLock()
    self.host: Dict[str, Timeline] = {}
    self.device: Dict[str, AsyncTimeline] = {}
    self.queued: Dict[str, Timeline] = {}

  def _get(self, table: Dict[str, Any], key: str, make: Callable[[str, float], Any]) -> Any:
    with self.lock:
      lane = table.get(key)
      if lane is None:
        lane = table[key] = make(key, self.born)
      return lane

  def host_lane(self, key: str) -> Timeline:
    return self._get(self.host, key, Timeline)

  def device_lane(self, key: str) -> AsyncTimeline:
    return self._get(self.device, key, AsyncTimeline)

  def queue_lane(self, key: str) -> Timeline:
    return self._get(self.queued, key, Timeline)

  def everything(self) -> Dict[str, Timeline]:
    with self.lock:
      return {**self.host, **self.device, **self.queued}

  def device_lanes(self) -> List[AsyncTimeline]:
    with self.lock:
      return list(self.device.values())


class PerfTracer(NoopTracer):

  def __init__(self, devices: Optional[Sequence[Any]] = None,
               export_fn: Optional[Callable[[Mapping[str, Timeline]], MetricsT]] = None,
               concurrent_spans: Union[None, str, Sequence[str]] = None,
               collect_on_first_device_per_mesh: bool = False):
    """`concurrent_spans`: span names that really overlap on a device (or "all"): device lanes that contain them
    are not split into active and queued parts."""
    self._export_fn = export_fn
    self._concurrent_spans = concurrent_spans
    self._collect_on_first_device_per_mesh = collect_on_first_device_per_mesh
    self._lanes = _Lanes(time.perf_counter())
    for lane_id in timeline_utils.generate_device_timeline_ids(devices):
      self._lanes.device_lane(lane_id)
    self._lanes.host_lane(timeline_utils.generate_host_timeline_id())

  def _get_timelines(self) -> Dict[str, Timeline]:
    return self._lanes.everything()

  @property
  def all_devices(self) -> Sequence[str]:
    with self._lanes.lock:
      return list(self._lanes.device)

  # ---- waiting and printing
  def synchronize(self) -> None:
    _synchronize_devices()
    for lane in self._lanes.device_lanes():
      lane.wait_pending_spans()

  def print(self) -> None:
    self.synchronize()
    for lane in self._get_timelines().values():
      print(repr(lane))

  # ---- end of step
  def _split_queued(self, lane_id: str, lane: AsyncTimeline) -> None:
    """Overlapping spans of a device lane are work that waited behind other work: the waiting part moves to the
    lane's queue timeline, the running parts stay and no longer overlap."""
    declared = self._concurrent_spans or []
    with lane._lock:
      if any(span.name in declared for span in lane._cur_step.values()):
        return
      running, waiting = timeline_utils.sequentialize_overlapping_spans(lane._cur_step)
      lane._cur_step = dict(running)
    if waiting:
      qlane = self._lanes.queue_lane(timeline_utils.generate_queued_timeline_id(lane_id))
      with qlane._lock:
        qlane._cur_step.update(waiting)

  def process_and_commit_timelines(self) -> None:
    with self._lanes.lock:
      for lane in self._lanes.device.values():
        lane.wait_pending_spans()
      if self._concurrent_spans != "all":
        for lane_id, lane in list(self._lanes.device.items()):
          self._split_queued(lane_id, lane)
      for lane in self._lanes.everything().values():
        lane.commit_step()

  def export(self) -> MetricsT:
    if self._export_fn is None:
      return {}
    self.process_and_commit_timelines()
    return self._export_fn(self._get_timelines())

  # ---- recording
  def _lanes_for(self, devices: Any) -> BatchAsyncTimelines:
    if self._collect_on_first_device_per_mesh and devices is not None:
      flat = devices.flatten().tolist() if isinstance(devices, np.ndarray) else list(devices)
      devices = flat[:1]
    return BatchAsyncTimelines([self._lanes.device_lane(lane_id)
                                for lane_id in timeline_utils.generate_device_timeline_ids(devices)])

  @contextlib.contextmanager
  def span(self, name: str, devices: Any = None, tags: Optional[Mapping[str, Any]] = None) -> Iterator[AsyncWaitlist]:
    issued_at = time.perf_counter()
    pending = AsyncWaitlist()
    host = self._lanes.host_lane(timeline_utils.generate_host_timeline_id())
    host.start_span(name, issued_at, tags=tags)
    try:
      yield pending
    finally:
      host.stop_span(time.perf_counter())
      self._lanes_for(devices).span(name, issued_at, pending.waitlist, tags=tags)


Tracer = Union[PerfTracer, NoopTracer]
