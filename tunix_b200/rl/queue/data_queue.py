"""Bounded hand-off queue between the rollout producer and the trainer
(tunix/rl/queue/data_queue.py:28-68)."""
from __future__ import annotations

import abc
import queue
from typing import Generic, Optional, TypeVar

T = TypeVar("T")


class AbstractDataQueue(abc.ABC, Generic[T]):

  @abc.abstractmethod
  def put(self, item: T) -> None:
    ...

  @abc.abstractmethod
  def get(self, block: bool = True, timeout: Optional[float] = None) -> T:
    ...

  @abc.abstractmethod
  def qsize(self) -> int:
    ...

  @abc.abstractmethod
  def close(self) -> None:
    ...


class SimpleDataQueue(AbstractDataQueue[T]):

  def __init__(self, maxsize: int = 0):
    self._queue: "queue.Queue[T]" = queue.Queue(maxsize=maxsize)

  def put(self, item: T) -> None:
    self._queue.put(item)

  def get(self, block: bool = True, timeout: Optional[float] = None) -> T:
    return self._queue.get(block=block, timeout=timeout)

  def qsize(self) -> int:
    return self._queue.qsize()

  def close(self) -> None:
    pass
