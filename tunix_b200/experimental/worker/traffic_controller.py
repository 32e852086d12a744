"""Admission gate of a rollout worker.

A rollout worker alternates between serving generation requests and receiving new weights. The
gate numbers those serving periods: epoch e is open while requests are admitted, a weight sync
closes it, and reopening starts epoch e + 1. Every admitted task carries the epoch it was admitted
in, so "drain before the weights change" is exactly "wait for the tasks of closed epochs" - tasks
admitted after a reopen never hold up a sync that was requested earlier, and nothing is polled.

The gate can be driven from any thread (the weight-sync RPC handler usually is not the event-loop
thread that runs the generation tasks): state lives under one mutex, and the only loop-affine
actions - cancelling a task, waking coroutines that wait for admission - are posted to the loop
that owns them.

Behaviour expected by callers (tunix/experimental/worker/traffic_controller.py:26-153): requests
are admitted only while READY; SYNCING closes admission and may be entered from READY or SYNCING
only; STOPPED is final and cancels everything in flight; a task refused admission is cancelled.
"""
from __future__ import annotations

import asyncio
import threading
from typing import Dict, List, Optional

from ..common import datatypes

WorkerState = datatypes.WorkerState


class AdmissionClosedError(RuntimeError):
  """A request arrived while the worker was not admitting (syncing, draining or stopped)."""


def _post(loop: asyncio.AbstractEventLoop, fn, *args) -> None:
  """Runs `fn(*args)` on `loop`: inline when already there, else through its thread-safe queue."""
  try:
    running = asyncio.get_running_loop()
  except RuntimeError:
    running = None
  if running is loop:
    fn(*args)
  elif not loop.is_closed():
    loop.call_soon_threadsafe(fn, *args)


class TrafficController:

  def __init__(self):
    self._home = asyncio.get_running_loop()       # loop of the coroutines that wait for admission
    self._mu = threading.Lock()
    self._phase = WorkerState.READY
    self._epoch = 0                               # number of the current (or last) serving period
    self._inflight: Dict[asyncio.Task, int] = {}  # task -> epoch of admission
    self._waiters: List[asyncio.Future] = []      # coroutines parked until the next READY

  # ---- observers ---------------------------------------------------------------------
  @property
  def state(self) -> WorkerState:
    return self._phase

  @property
  def epoch(self) -> int:
    return self._epoch

  def is_admission_open(self) -> bool:
    return self._phase == WorkerState.READY

  def get_active_tasks(self) -> List[asyncio.Task]:
    with self._mu:
      return list(self._inflight)

  async def wait_for_admission(self) -> None:
    """Returns once requests are admitted again (at once when they are)."""
    with self._mu:
      if self._phase == WorkerState.READY:
        return
      fut = self._home.create_future()
      self._waiters.append(fut)
    await fut

  # ---- admission ----------------------------------------------------------------------
  def track(self, task: asyncio.Task) -> None:
    """Counts `task` as in flight in the current epoch, whatever the phase."""
    with self._mu:
      self._inflight[task] = self._epoch
    task.add_done_callback(self._forget)

  def try_admit(self, task: asyncio.Task) -> bool:
    """Admits `task` while READY; otherwise cancels it and reports False."""
    with self._mu:
      admitted = self._phase == WorkerState.READY
      if admitted:
        self._inflight[task] = self._epoch
    if admitted:
      task.add_done_callback(self._forget)
    else:
      _post(task.get_loop(), task.cancel)
    return admitted

  def _forget(self, task: asyncio.Task) -> None:
    with self._mu:
      self._inflight.pop(task, None)

  # ---- phase changes --------------------------------------------------------------------
  def transition_to_syncing(self) -> None:
    with self._mu:
      if self._phase == WorkerState.STOPPED or self._phase not in (WorkerState.READY, WorkerState.SYNCING):
        raise RuntimeError(f"Cannot transition to SYNCING from {self._phase.value}")
      self._phase = WorkerState.SYNCING          # the current epoch is now closed

  async def drain(self, timeout_s: Optional[float]) -> None:
    """Waits (at most `timeout_s`) for the tasks admitted up to the current epoch."""
    with self._mu:
      old = [t for t, e in self._inflight.items() if e <= self._epoch]
    if old:
      await asyncio.wait(old, timeout=timeout_s)

  def reopen(self) -> bool:
    """Starts the next serving epoch; False when the worker was stopped for good."""
    with self._mu:
      if self._phase == WorkerState.STOPPED:
        return False
      if self._phase != WorkerState.READY:
        self._epoch += 1
      self._phase = WorkerState.READY
      parked, self._waiters = self._waiters, []
    for fut in parked:
      _post(self._home, lambda f=fut: f.done() or f.set_result(None))
    return True

  def stop_and_cancel_all(self) -> List[asyncio.Task]:
    with self._mu:
      self._phase = WorkerState.STOPPED
      doomed = list(self._inflight)
    for t in doomed:
      _post(t.get_loop(), t.cancel)
    return doomed
