"""Spans and timelines (tunix/perf/experimental/timeline.py:32-410).

A `Timeline` records the nested spans of one host thread; `commit_step` archives the finished spans of a step
(the list of committed steps is replaced, never mutated, so readers take no lock) and drops spans that are still
open. An `AsyncTimeline` is a device lane: a span there begins when the host issued the work and ends when the
work is done on the device.

How "done on the device" is observed. The reference parks one waiter thread per span on the arrays' readiness and
stamps the host clock when it wakes up. Here a span's end is a *completion* object:

  * for CUDA work (a tensor, a `torch.cuda.Event`, a stream) `span()` records a timing event on the device's
    current stream - everything issued so far, hence the work the waitlist names - and the end time is read back
    later as `anchor host time + elapsed(anchor event, end event)`, i.e. a device timestamp with no thread wake-up
    in it. Nothing blocks and no thread exists until somebody asks for the spans (`wait_pending_spans`);
  * for anything else that can be waited on (`synchronize()` / `result()` / `wait()`: futures, handles of other
    runtimes) one resolver thread per timeline takes the waits in order and stamps the host clock.
"""
from __future__ import annotations

import dataclasses
import itertools
import logging
import queue
import threading
import time
from typing import Any, Dict, Iterable, Iterator, List, Mapping, Optional, Tuple

log = logging.getLogger(__name__)
_INF = float("inf")


@dataclasses.dataclass
class Span:
  name: str
  begin: float
  id: int
  end: float = dataclasses.field(default=_INF, init=False)
  parent_id: Optional[int] = None
  tags: Optional[Mapping[str, Any]] = None

  def __post_init__(self) -> None:
    self.tags = {} if self.tags is None else dict(self.tags)

  @property
  def ended(self) -> bool:
    return self.end != _INF

  @property
  def duration(self) -> float:
    return self.end - self.begin

  def add_tag(self, key: str, value: Any) -> None:
    if key in self.tags:
      log.warning("Span '%s' (id=%s): tag %r already set to %r; overwriting with %r", self.name, self.id, key,
                  self.tags[key], value)
    self.tags[key] = value

  def _format_relative(self, born_at: float) -> str:
    parent = "" if self.parent_id is None else f" (parent={self.parent_id})"
    tags = f", tags={self.tags}" if self.tags else ""
    return f"[{self.id}] {self.name}: {self.begin - born_at:.6f}, {self.end - born_at:.6f}{parent}{tags}"


# ------------------------------------------------------------------------------------ waitables
def _leaves(waitlist: Any) -> Iterator[Any]:
  """Flattens nestings of mappings / sequences / sets into the things that can be waited on."""
  if waitlist is None:
    return
  if isinstance(waitlist, Mapping):
    waitlist = list(waitlist.values())
  if isinstance(waitlist, (list, tuple, set)):
    for item in waitlist:
      yield from _leaves(item)
    return
  yield waitlist


def _cuda_device_of(item: Any) -> Optional[int]:
  """Device index if `item` is CUDA work this process can time with events, else None."""
  try:
    import torch
  except ImportError:       # pragma: no cover
    return None
  if isinstance(item, torch.Tensor):
    return item.device.index if item.is_cuda else None
  if isinstance(item, (torch.cuda.Event, torch.cuda.Stream)):
    return getattr(item, "device", torch.device("cuda", torch.cuda.current_device())).index
  return None


def wait_for(waitlist: Any) -> None:
  """Blocks until everything in `waitlist` is done: CUDA events, tensors (their device's current work), objects
  with `synchronize()` / `result()` / `wait()`, or nestings of those."""
  for item in _leaves(waitlist):
    dev = _cuda_device_of(item)
    if dev is not None:
      import torch
      if isinstance(item, torch.Tensor):
        torch.cuda.synchronize(dev)
      else:
        item.synchronize()
      continue
    for verb in ("synchronize", "result", "wait"):
      call = getattr(item, verb, None)
      if callable(call):
        call()
        break


class _DeviceClock:
  """Maps CUDA event times of one device onto the host's `perf_counter` axis through an anchor pair taken once."""

  _by_device: Dict[int, "_DeviceClock"] = {}
  _guard = threading.Lock()

  def __init__(self, device: int):
    import torch
    self.device = device
    with torch.cuda.device(device):
      torch.cuda.synchronize(device)
      self.anchor = torch.cuda.Event(enable_timing=True)
      self.anchor.record()
      self.anchor.synchronize()
    self.anchor_host = time.perf_counter()

  @classmethod
  def of(cls, device: int) -> "_DeviceClock":
    with cls._guard:
      clock = cls._by_device.get(device)
      if clock is None:
        clock = cls._by_device[device] = cls(device)
      return clock

  def mark(self):
    """A timing event on the device's current stream, recorded now."""
    import torch
    with torch.cuda.device(self.device):
      ev = torch.cuda.Event(enable_timing=True)
      ev.record()
    return ev

  def host_time(self, ev) -> float:
    ev.synchronize()
    return self.anchor_host + self.anchor.elapsed_time(ev) * 1e-3


# ------------------------------------------------------------------------------------ host timeline
class Timeline:

  def __init__(self, id: str, born: float):
    self.id = id
    self.born = born
    self._lock = threading.RLock()
    self._ids = itertools.count()
    self._spans_stack: List[int] = []                  # ids of the open spans, innermost last
    self._cur_step: Dict[int, Span] = {}
    self._committed_steps: List[Dict[int, Span]] = []

  # ---- views
  @property
  def committed_steps(self) -> List[Dict[int, Span]]:
    return self._committed_steps

  @property
  def cur_step(self) -> Dict[int, Span]:
    with self._lock:
      return dict(self._cur_step)

  @property
  def all_steps(self) -> List[Dict[int, Span]]:
    with self._lock:
      return [*self._committed_steps, dict(self._cur_step)]

  # ---- recording
  def _new_span(self, name: str, begin: float, tags: Optional[Mapping[str, Any]]) -> Span:
    """A span under the innermost open one. Caller holds the lock."""
    return Span(name=name, begin=begin, id=next(self._ids), tags=tags,
                parent_id=self._spans_stack[-1] if self._spans_stack else None)

  def start_span(self, name: str, begin: float, tags: Optional[Mapping[str, Any]] = None) -> Span:
    with self._lock:
      span = self._new_span(name, begin, tags)
      self._cur_step[span.id] = span
      self._spans_stack.append(span.id)
      return span

  def stop_span(self, end: float) -> None:
    with self._lock:
      if not self._spans_stack:
        raise ValueError(f"{self.id}: no more spans to end.")
      span = self._cur_step[self._spans_stack.pop()]
      if end < span.begin:
        raise ValueError(f"{self.id}: span '{span.name}' ended at {end:.6f} before it began at {span.begin:.6f}.")
      span.end = end

  def commit_step(self) -> None:
    """Archives the finished spans of the current step; spans still open (or never ended) are dropped."""
    with self._lock:
      still_open = set(self._spans_stack)
      kept: Dict[int, Span] = {}
      for sid, span in self._cur_step.items():
        if span.ended and sid not in still_open:
          kept[sid] = span
        else:
          log.warning("Purging uncompleted span %r crossing step boundary in timeline %s", span.name, self.id)
      self._spans_stack.clear()
      self._committed_steps = [*self._committed_steps, kept]
      self._cur_step = {}

  def __repr__(self) -> str:
    lines = [f"Timeline({self.id}, {self.born:.6f})"]
    for number, step in enumerate(self.all_steps):
      lines.append(f"  step {number}:")
      lines.extend(f"    {span._format_relative(self.born)}" for span in step.values())
    return "\n".join(lines) + "\n"


# ------------------------------------------------------------------------------------ device lane
class AsyncTimeline(Timeline):

  def __init__(self, id: str, born: float):
    super().__init__(id, born)
    self._device_marks: List[Tuple[Span, List[Tuple[_DeviceClock, Any]]]] = []     # spans closed by CUDA events
    self._host_waits: "queue.Queue[Optional[Tuple[Span, List[Any]]]]" = queue.Queue()
    self._resolver: Optional[threading.Thread] = None

  # ---- the resolver thread for non-CUDA waitables (started on first use)
  def _resolve_host_waits(self) -> None:
    while True:
      job = self._host_waits.get()
      try:
        if job is None:
          return
        span, items = job
        try:
          wait_for(items)
        except Exception as e:  # noqa: BLE001 - a failed wait loses one span, not the tracer
          log.error("Timeline span '%s' (id=%d) failed: %s", span.name, span.id, e)
          continue
        self._close(span, time.perf_counter())
      finally:
        self._host_waits.task_done()

  def _close(self, span: Span, end: float) -> None:
    span.end = max(end, span.begin)
    with self._lock:
      self._cur_step[span.id] = span

  def span(self, name: str, thread_span_begin: float, waitlist: Any,
           tags: Optional[Mapping[str, Any]] = None) -> None:
    """A span from `thread_span_begin` (host time at which the work was issued) to the completion of `waitlist`."""
    with self._lock:
      span = self._new_span(name, thread_span_begin, tags)
    marks: List[Tuple[_DeviceClock, Any]] = []
    others: List[Any] = []
    for item in _leaves(waitlist):
      dev = _cuda_device_of(item)
      if dev is None:
        others.append(item)
      else:
        marks.append((_DeviceClock.of(dev), _DeviceClock.of(dev).mark()))
    if not marks and not others:
      self._close(span, time.perf_counter())
      return
    if others:
      # host-side waits decide the end; device marks (if any) are waited for by the same resolver
      with self._lock:
        if self._resolver is None:
          self._resolver = threading.Thread(target=self._resolve_host_waits, daemon=True, name=f"perf-lane-{self.id}")
          self._resolver.start()
      self._host_waits.put((span, others + [ev for _, ev in marks]))
      return
    with self._lock:
      self._device_marks.append((span, marks))

  def wait_pending_spans(self) -> None:
    """Returns once every span issued so far has its end time."""
    with self._lock:
      marked, self._device_marks = self._device_marks, []
    for span, marks in marked:
      try:
        self._close(span, max(clock.host_time(ev) for clock, ev in marks))
      except Exception as e:  # noqa: BLE001
        log.error("Timeline span '%s' (id=%d) failed: %s", span.name, span.id, e)
    if self._resolver is not None:
      self._host_waits.join()


class BatchAsyncTimelines:
  """The same span on several device lanes."""

  def __init__(self, timelines: Iterable[AsyncTimeline]):
    self._timelines = list(timelines)

  def span(self, name: str, thread_span_begin: float, waitlist: Any,
           tags: Optional[Mapping[str, Any]] = None) -> None:
    for lane in self._timelines:
      lane.span(name, thread_span_begin, waitlist, tags=tags)
