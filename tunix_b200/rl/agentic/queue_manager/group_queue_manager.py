"""Groups trajectories and releases them in training batches.

Asynchronous rollouts finish one trajectory at a time and in any order, while group-relative
algorithms need all G samples of a prompt together. This queue has two halves:

  * an *assembler* that holds unfinished groups - by default keyed buckets of `group_size` items
    (`key_fn(item)` names the bucket), or any callable `group_fn(buckets, item)` that returns a
    finished group or None;
  * an *outbox*: a FIFO of single items. A finished group that survives `filter_fn` is appended to
    it as a run of consecutive items, so `get_batch(n)` is simply "take the next n items" and a
    group that straddles two batches continues at the head of the next one without any splitting
    bookkeeping.

One `asyncio.Condition` guards all state and wakes consumers; producers never block. A producer's
failure (`put_exception`) poisons the queue: every later `put` and `get_batch` raises it until
`clear()`. `prepare_clear()` turns the queue into a drain - puts are dropped, waiting consumers
return with what they have - so a learner can stop a generation wave between steps.

Behaviour follows tunix/rl/agentic/queue_manager/group_queue_manager.py:37-205.
"""
from __future__ import annotations

import asyncio
import collections
from typing import Any, Callable, Deque, Dict, Generic, Hashable, List, Optional, Tuple, TypeVar, Union

T = TypeVar("T")
GroupFn = Callable[[Dict[Hashable, List[T]], T], Optional[List[T]]]
FilterFn = Callable[[List[T]], Union[List[T], Tuple[List[T], List[T]]]]


class _CountByKey(Generic[T]):
  """Default assembler: a group is `size` items that share `key(item)`."""

  def __init__(self, size: int, key: Callable[[T], Hashable]):
    self.size, self.key = size, key

  def __call__(self, buckets: Dict[Hashable, List[T]], item: T) -> Optional[List[T]]:
    k = self.key(item)
    members = buckets[k]
    members.append(item)
    return buckets.pop(k) if len(members) >= self.size else None


class GroupQueueManager(Generic[T]):

  def __init__(self, *, group_size: Optional[int] = None, key_fn: Optional[Callable[[T], Hashable]] = None,
               group_fn: Optional[GroupFn] = None, filter_fn: Optional[FilterFn] = None):
    if group_fn is None:
      if group_size is None:
        raise ValueError("GroupQueueManager needs `group_size` (with an optional `key_fn`) or a custom `group_fn`")
      group_fn = _CountByKey(group_size, key_fn or id)
    self.group_size, self.group_fn, self.filter_fn = group_size, group_fn, filter_fn
    self._open_groups: Dict[Hashable, List[T]] = collections.defaultdict(list)
    self._outbox: Deque[T] = collections.deque()
    self._runs: Deque[int] = collections.deque()      # lengths of the groups that make up the outbox, in order
    self._rejected: List[List[T]] = []
    self._draining = False
    self._poison: Optional[BaseException] = None
    self._changed = asyncio.Condition()

  # ---- producer side ------------------------------------------------------------------
  def _split_by_filter(self, group: List[T]) -> Tuple[List[T], List[T]]:
    if self.filter_fn is None:
      return group, []
    verdict = self.filter_fn(group)
    if isinstance(verdict, tuple) and len(verdict) == 2:
      return list(verdict[0]), list(verdict[1])
    kept = list(verdict)
    kept_ids = {id(x) for x in kept}
    return kept, [x for x in group if id(x) not in kept_ids]

  async def put(self, item: T) -> None:
    async with self._changed:
      if self._draining:
        return
      if self._poison is not None:
        raise self._poison
      group = self.group_fn(self._open_groups, item)
      if group is None:
        return
      kept, dropped = self._split_by_filter(group)
      if dropped:
        self._rejected.append(dropped)
      if kept:
        self._outbox.extend(kept)
        self._runs.append(len(kept))
        self._changed.notify_all()

  async def put_exception(self, exc: BaseException) -> None:
    async with self._changed:
      self._poison = exc
      self._changed.notify_all()

  # ---- consumer side --------------------------------------------------------------------
  async def get_batch(self, batch_size: int) -> List[T]:
    """The next `batch_size` items in release order; waits for them. Returns fewer (possibly none) only when
    the queue is being cleared."""
    out: List[T] = []
    async with self._changed:
      while True:
        if self._poison is not None:
          raise self._poison
        while self._outbox and len(out) < batch_size:
          out.append(self._take_one())
        if len(out) >= batch_size or self._draining:
          return out
        await self._changed.wait()

  def _take_one(self) -> T:
    self._runs[0] -= 1
    if self._runs[0] == 0:
      self._runs.popleft()
    return self._outbox.popleft()

  async def get_group(self) -> List[T]:
    """The next whole group in release order (what is left of it, if `get_batch` already took its head); waits
    for one. Empty only when the queue is being cleared."""
    async with self._changed:
      while True:
        if self._poison is not None:
          raise self._poison
        if self._runs:
          return [self._take_one() for _ in range(self._runs[0])]
        if self._draining:
          return []
        await self._changed.wait()

  async def get_filtered_groups(self) -> List[List[T]]:
    """Groups (or parts of groups) the filter rejected since the last call."""
    async with self._changed:
      out, self._rejected = self._rejected, []
      return out

  # ---- lifecycle ---------------------------------------------------------------------------
  async def prepare_clear(self) -> None:
    async with self._changed:
      self._draining = True
      self._changed.notify_all()

  async def clear(self) -> None:
    async with self._changed:
      self._open_groups.clear()
      self._outbox.clear()
      self._runs.clear()
      self._rejected = []
      self._poison, self._draining = None, False
