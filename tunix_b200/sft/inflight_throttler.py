"""Bounds how many training steps may be queued on the GPU ahead of the host.

The host enqueues kernels asynchronously; without a bound it can run arbitrarily far ahead
(pinning batches and metric tensors). Each step hands the throttler a CUDA event (or any
object with `synchronize()`/`wait()`), and `wait_for_next` blocks on the oldest one once
`max_inflight` are outstanding (tunix/sft/inflight_throttler.py:21-67).
"""
from __future__ import annotations

import collections
from typing import Any, Deque

import torch


def _block(obj: Any) -> None:
  if obj is None:
    return
  if isinstance(obj, torch.cuda.Event):
    obj.synchronize()
  elif isinstance(obj, torch.Tensor):
    if obj.is_cuda:
      torch.cuda.current_stream(obj.device).synchronize()
  elif hasattr(obj, "synchronize"):
    obj.synchronize()
  elif hasattr(obj, "wait"):
    obj.wait()


class InflightThrottler:

  def __init__(self, max_inflight: int):
    self._max_inflight = max_inflight
    self._queue: Deque[Any] = collections.deque()

  def add_computation(self, computation: Any) -> None:
    if self._max_inflight is None or self._max_inflight < 0:
      return
    if isinstance(computation, torch.Tensor) and computation.is_cuda:
      ev = torch.cuda.Event()
      ev.record(torch.cuda.current_stream(computation.device))
      computation = ev
    self._queue.append(computation)

  def wait_for_next(self) -> None:
    if self._max_inflight is None or self._max_inflight < 0:
      return
    while len(self._queue) > self._max_inflight:
      _block(self._queue.popleft())

  def wait_for_all(self) -> None:
    while self._queue:
      _block(self._queue.popleft())

  def __len__(self) -> int:
    return len(self._queue)
