"""Async grouping queue (tunix/rl/agentic/queue_manager/group_queue_manager.py:37-205).

Items are bucketed by a key until a bucket holds `group_size` items (or a custom `group_fn`
says a group is complete); complete groups pass an optional filter and are handed out in
batches. A producer failure is stored and re-raised to every later `put` / `get_batch`.
"""
from __future__ import annotations

import asyncio
import collections
from typing import Any, Callable, Deque, Dict, Generic, Hashable, List, Optional, Tuple, TypeVar, Union

T = TypeVar("T")
GroupFn = Callable[[Dict[Hashable, List[T]], T], Optional[List[T]]]
FilterFn = Callable[[List[T]], Union[List[T], Tuple[List[T], List[T]]]]


class GroupQueueManager(Generic[T]):
  def __init__(self, *, group_size: Optional[int] = None, key_fn: Optional[Callable[[T], Hashable]] = None,
               group_fn: Optional[GroupFn] = None, filter_fn: Optional[FilterFn] = None):
    if group_fn is None:
      if group_size is None:
        raise ValueError("Must specify either group_size or a custom group_fn for GroupQueueManager.")
      key = key_fn or id

      def group_fn(buckets, item):
        k = key(item)
        buckets[k].append(item)
        if len(buckets[k]) == group_size:
          return buckets.pop(k)
        return None
    self.group_size, self.group_fn, self.filter_fn = group_size, group_fn, filter_fn
    self._buckets: Dict[Hashable, List[T]] = collections.defaultdict(list)
    self._ready: Deque[List[T]] = collections.deque()
    self._filtered: Deque[List[T]] = collections.deque()
    self._clearing = False
    self._exc: Optional[BaseException] = None
    self._lock = asyncio.Lock()
    self._have_ready = asyncio.Event()

  async def put_exception(self, exc: BaseException) -> None:
    self._exc = exc
    self._have_ready.set()

  async def prepare_clear(self) -> None:
    self._clearing = True
    self._have_ready.set()

  async def clear(self) -> None:
    async with self._lock:
      self._buckets.clear()
      self._ready.clear()
      self._filtered.clear()
      self._exc, self._clearing = None, False
      self._have_ready.clear()

  async def get_filtered_groups(self) -> List[List[T]]:
    async with self._lock:
      out = list(self._filtered)
      self._filtered.clear()
      return out

  def _apply_filter(self, group: List[T]) -> Tuple[List[T], List[T]]:
    if self.filter_fn is None:
      return group, []
    res = self.filter_fn(group)
    if isinstance(res, tuple) and len(res) == 2:
      return res
    kept = {id(x) for x in res}
    return list(res), [x for x in group if id(x) not in kept]

  async def put(self, item: T) -> None:
    if self._clearing:
      return
    if self._exc:
      raise self._exc
    async with self._lock:
      if self._clearing:
        return
      if self._exc:
        raise self._exc
      group = self.group_fn(self._buckets, item)
      if group is None:
        return
      valid, dropped = self._apply_filter(group)
      if dropped:
        self._filtered.append(dropped)
      if valid:
        self._ready.append(valid)
        self._have_ready.set()

  async def _next_group(self) -> List[T]:
    while True:
      if self._exc:
        raise self._exc
      if self._clearing:
        return []
      async with self._lock:
        if self._ready:
          return self._ready.popleft()
      await self._have_ready.wait()
      self._have_ready.clear()

  async def get_batch(self, batch_size: int) -> List[T]:
    """Waits until `batch_size` items are available (fewer only when clearing). A group that
    does not fit is split and its remainder goes back to the front."""
    out: List[T] = []
    while len(out) < batch_size:
      group = await self._next_group()
      if not group:
        break
      async with self._lock:
        room = batch_size - len(out)
        out.extend(group[:room])
        if len(group) > room:
          self._ready.appendleft(group[room:])
          self._have_ready.set()
    return out
