"""Admission control of a rollout worker (tunix/experimental/worker/traffic_controller.py:26-153).

One object owns the worker's serving state and the set of running generation tasks: requests
are admitted only while READY; a weight sync closes admission (SYNCING), waits for or cancels
the tasks in flight, and reopens afterwards; STOPPED is final. State changes may come from
another thread than the event loop that runs the tasks, so loop-affine operations are posted
to the loop."""
from __future__ import annotations

import asyncio
import threading
from typing import Any, List, Set

from ..common import datatypes

WorkerState = datatypes.WorkerState


class AdmissionClosedError(RuntimeError):
  """A request arrived while the worker was not admitting (syncing, draining or stopped)."""


class TrafficController:
  def __init__(self):
    self._loop = asyncio.get_running_loop()
    self._lock = threading.RLock()
    self._state = WorkerState.READY
    self._open = asyncio.Event()
    self._open.set()
    self._tasks: Set[asyncio.Task] = set()

  def _on_loop(self, loop: asyncio.AbstractEventLoop, fn) -> None:
    try:
      here = asyncio.get_running_loop()
    except RuntimeError:
      here = None
    fn() if here is loop else loop.call_soon_threadsafe(fn)

  @property
  def state(self) -> WorkerState:
    with self._lock:
      return self._state

  async def wait_for_admission(self) -> None:
    await self._open.wait()

  def is_admission_open(self) -> bool:
    with self._lock:
      return self._state == WorkerState.READY and self._open.is_set()

  def try_admit(self, task: asyncio.Task) -> bool:
    """Tracks the task when READY; otherwise cancels it and returns False."""
    with self._lock:
      if self._state != WorkerState.READY:
        self._on_loop(task.get_loop(), task.cancel)
        return False
      self.track(task)
      return True

  def track(self, task: asyncio.Task) -> None:
    with self._lock:
      self._tasks.add(task)
    task.add_done_callback(self._done)

  def _done(self, task: asyncio.Task) -> None:
    with self._lock:
      self._tasks.discard(task)

  def get_active_tasks(self) -> List[asyncio.Task]:
    with self._lock:
      return list(self._tasks)

  async def drain(self, timeout_s: float) -> None:
    tasks = self.get_active_tasks()
    if tasks:
      await asyncio.wait(tasks, timeout=timeout_s)

  def transition_to_syncing(self) -> None:
    with self._lock:
      if self._state not in (WorkerState.READY, WorkerState.SYNCING):
        raise RuntimeError(f"Cannot transition to SYNCING from {self._state.value}")
      self._state = WorkerState.SYNCING
      self._on_loop(self._loop, self._open.clear)

  def reopen(self) -> bool:
    with self._lock:
      if self._state == WorkerState.STOPPED:
        return False
      self._state = WorkerState.READY
      self._on_loop(self._loop, self._open.set)
      return True

  def stop_and_cancel_all(self) -> List[asyncio.Task]:
    with self._lock:
      self._state = WorkerState.STOPPED
      self._on_loop(self._loop, self._open.clear)
      tasks = list(self._tasks)
    for t in tasks:
      self._on_loop(t.get_loop(), t.cancel)
    return tasks
