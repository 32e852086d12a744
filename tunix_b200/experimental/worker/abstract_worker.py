"""Worker interface with a validated lifecycle (tunix/experimental/worker/abstract_worker.py:28-86):
PENDING -> INITIALIZING -> READY <-> {COMPILING, SYNCING} -> DRAINING -> STOPPED, ERROR from
anywhere; an illegal transition raises instead of silently corrupting the state."""
from __future__ import annotations

import abc
import contextlib
import threading
from typing import Any

from ..common import datatypes


class Worker(abc.ABC):
  _state: datatypes.WorkerState = datatypes.WorkerState.PENDING

  @property
  def state(self) -> datatypes.WorkerState:
    return self._state

  @state.setter
  def state(self, new_state: datatypes.WorkerState) -> None:
    if self._state == new_state:
      return
    if not self._state.can_transition_to(new_state):
      raise RuntimeError(f"Invalid transition from {self._state.name} to {new_state.name}")
    self._state = new_state

  @contextlib.contextmanager
  def _phase(self, during: datatypes.WorkerState, after: datatypes.WorkerState = datatypes.WorkerState.READY):
    """State is `during` inside the block, `after` on success, ERROR when the block raises."""
    self.state = during
    try:
      yield
    except BaseException:
      self._state = datatypes.WorkerState.ERROR
      raise
    self.state = after

  @abc.abstractmethod
  def initialize(self) -> datatypes.Response: ...

  @abc.abstractmethod
  def compile(self, dummy_data: Any) -> datatypes.Response: ...

  @abc.abstractmethod
  def start(self) -> datatypes.Response: ...

  @abc.abstractmethod
  def stop(self) -> datatypes.Response: ...

  @abc.abstractmethod
  def info(self) -> datatypes.WorkerInfo: ...

  @abc.abstractmethod
  def heartbeat(self) -> datatypes.HealthReport: ...
