"""Hand-off queue between the rollout producer thread and the training loop.

The producer generates, scores and annotates micro-batches while the trainer consumes earlier ones;
the queue's capacity is what bounds how far generation may run ahead of the policy that trains on it.
Unlike a plain `queue.Queue`, `close()` wakes every blocked producer and consumer - a learner that
stops early (an exception in the training loop, `max_steps` reached) never leaves the other thread
parked forever: blocked `put`s are dropped, blocked `get`s raise `QueueClosed`.

Interface of tunix/rl/queue/data_queue.py:28-68 (`put`, `get`, `qsize`, `close`).
"""
from __future__ import annotations

import abc
import collections
import threading
import time
from typing import Deque, Generic, Optional, TypeVar

T = TypeVar("T")


class QueueClosed(RuntimeError):
  """`get` on a queue that was closed while (or before) waiting and holds nothing more."""


class AbstractDataQueue(abc.ABC, Generic[T]):
  """What the learners need from a producer/consumer channel."""

  @abc.abstractmethod
  def put(self, item: T) -> None:
    """Appends `item`, waiting while the queue is full."""

  @abc.abstractmethod
  def get(self, block: bool = True, timeout: Optional[float] = None) -> T:
    """Removes and returns the oldest item."""

  @abc.abstractmethod
  def qsize(self) -> int:
    """Items currently held."""

  @abc.abstractmethod
  def close(self) -> None:
    """No more traffic: releases every waiter."""


class SimpleDataQueue(AbstractDataQueue[T]):
  """In-process FIFO with an optional capacity (`maxsize` <= 0: unbounded)."""

  def __init__(self, maxsize: int = 0):
    self._cap = maxsize if maxsize and maxsize > 0 else None
    self._items: Deque[T] = collections.deque()
    self._cv = threading.Condition()
    self._closed = False

  def put(self, item: T) -> None:
    with self._cv:
      while self._cap is not None and len(self._items) >= self._cap and not self._closed:
        self._cv.wait()
      if self._closed:
        return
      self._items.append(item)
      self._cv.notify_all()

  def get(self, block: bool = True, timeout: Optional[float] = None) -> T:
    deadline = None if timeout is None else time.monotonic() + timeout
    with self._cv:
      while not self._items:
        if self._closed:
          raise QueueClosed("the data queue was closed")
        if not block:
          raise IndexError("the data queue is empty")
        left = None if deadline is None else deadline - time.monotonic()
        if left is not None and left <= 0:
          raise TimeoutError("no item arrived in time")
        self._cv.wait(left)
      item = self._items.popleft()
      self._cv.notify_all()
      return item

  def qsize(self) -> int:
    with self._cv:
      return len(self._items)

  def close(self) -> None:
    with self._cv:
      self._closed = True
      self._cv.notify_all()
