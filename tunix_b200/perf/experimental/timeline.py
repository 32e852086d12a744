"""Spans and timelines (tunix/perf/experimental/timeline.py:32-410).

A `Timeline` records nested spans of one host thread; `commit_step` archives the finished spans
of a step (copy-on-write, so readers of committed steps take no lock) and drops spans that are
still open. An `AsyncTimeline` is a device lane: its spans begin when the host issued the work
and end when a waiter thread sees the work's CUDA events (or tensors' producing streams)
complete.
"""
from __future__ import annotations

import dataclasses
import logging
import threading
import time
from typing import Any, Callable, Dict, Iterable, List, Mapping, Optional

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
    self.tags = dict(self.tags) if self.tags is not None else {}

  def add_tag(self, key: str, value: Any) -> None:
    if key in self.tags:
      log.warning("Span '%s' (id=%s): tag %r already set to %r; overwriting with %r", self.name, self.id, key,
                  self.tags[key], value)
    self.tags[key] = value

  def _format_relative(self, born_at: float) -> str:
    out = f"[{self.id}] {self.name}: {self.begin - born_at:.6f}, {self.end - born_at:.6f}"
    if self.parent_id is not None:
      out += f" (parent={self.parent_id})"
    if self.tags:
      out += f", tags={self.tags}"
    return out

  @property
  def ended(self) -> bool:
    return self.end != _INF

  @property
  def duration(self) -> float:
    return self.end - self.begin


def wait_for(waitlist: Any) -> None:
  """Blocks until everything in `waitlist` is done: CUDA events, tensors (their device's current
  work), objects with `synchronize()` / `result()` / `wait()`, or nestings of those."""
  if waitlist is None:
    return
  if isinstance(waitlist, Mapping):
    for v in waitlist.values():
      wait_for(v)
    return
  if isinstance(waitlist, (list, tuple, set)):
    for v in waitlist:
      wait_for(v)
    return
  try:
    import torch
    if isinstance(waitlist, torch.Tensor):
      if waitlist.is_cuda:
        torch.cuda.synchronize(waitlist.device)
      return
  except ImportError:   # pragma: no cover
    pass
  for attr in ("synchronize", "result", "wait"):
    fn = getattr(waitlist, attr, None)
    if callable(fn):
      fn()
      return


def _async_wait(waitlist: Any, success: Callable[[], None], failure: Callable[[Exception], None]) -> threading.Thread:
  def run():
    try:
      wait_for(waitlist)
    except Exception as e:  # pylint: disable=broad-exception-caught
      failure(e)
      return
    success()
  t = threading.Thread(target=run, daemon=True, name="perf-span-wait")
  t.start()
  return t


class Timeline:

  def __init__(self, id: str, born: float):
    self.id = id
    self.born = born
    self._spans_stack: List[int] = []
    self._cur_step: Dict[int, Span] = {}
    self._last_span_id = -1
    self._committed_steps: List[Dict[int, Span]] = []
    self._lock = threading.RLock()

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
      return self._committed_steps + [dict(self._cur_step)]

  def start_span(self, name: str, begin: float, tags: Optional[Mapping[str, Any]] = None) -> Span:
    with self._lock:
      parent = self._spans_stack[-1] if self._spans_stack else None
      self._last_span_id += 1
      span = Span(name=name, begin=begin, id=self._last_span_id, parent_id=parent, tags=tags)
      self._cur_step[span.id] = span
      self._spans_stack.append(span.id)
    return span

  def stop_span(self, end: float) -> None:
    with self._lock:
      if not self._spans_stack:
        raise ValueError(f"{self.id}: no more spans to end.")
      span = self._cur_step[self._spans_stack.pop()]
      if span.begin > end:
        raise ValueError(f"{self.id}: span '{span.name}' ended at {end:.6f} before it began at {span.begin:.6f}.")
      span.end = end

  def commit_step(self) -> None:
    with self._lock:
      for sid in [s for s, sp in self._cur_step.items() if not sp.ended or s in self._spans_stack]:
        log.warning("Purging uncompleted span %r crossing step boundary in timeline %s", self._cur_step[sid].name,
                    self.id)
        self._cur_step.pop(sid, None)
      self._spans_stack.clear()
      self._committed_steps = list(self._committed_steps) + [self._cur_step]
      self._cur_step = {}

  def __repr__(self) -> str:
    lines = [f"Timeline({self.id}, {self.born:.6f})"]
    for i, step in enumerate(self.all_steps):
      lines.append(f"  step {i}:")
      lines += [f"    {sp._format_relative(self.born)}" for sp in step.values()]
    return "\n".join(lines) + "\n"


class AsyncTimeline(Timeline):

  def __init__(self, id: str, born: float):
    super().__init__(id, born)
    self._threads: List[threading.Thread] = []

  def span(self, name: str, thread_span_begin: float, waitlist: Any,
           tags: Optional[Mapping[str, Any]] = None) -> None:
    with self._lock:
      parent = self._spans_stack[-1] if self._spans_stack else None
      self._last_span_id += 1
      sid = self._last_span_id

    def on_success() -> None:
      end = time.perf_counter()
      with self._lock:
        sp = Span(name=name, begin=thread_span_begin, id=sid, parent_id=parent, tags=tags)
        sp.end = end
        self._cur_step[sid] = sp

    def on_failure(e: Exception) -> None:
      log.error("Timeline span '%s' (id=%d) failed: %s", name, sid, e)

    if not waitlist:
      on_success()
      return
    t = _async_wait(waitlist, on_success, on_failure)
    with self._lock:
      self._threads = [x for x in self._threads if x.is_alive()] + [t]

  def wait_pending_spans(self) -> None:
    with self._lock:
      threads, self._threads = list(self._threads), []
    for t in threads:
      t.join()


class BatchAsyncTimelines:

  def __init__(self, timelines: Iterable[AsyncTimeline]):
    self._timelines = list(timelines)

  def span(self, name: str, thread_span_begin: float, waitlist: Any,
           tags: Optional[Mapping[str, Any]] = None) -> None:
    for tl in self._timelines:
      tl.span(name, thread_span_begin, waitlist, tags=tags)
