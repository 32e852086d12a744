"""Worker double for orchestration tests (tunix/experimental/worker/mock_worker.py:26-98): counts
calls, optionally appends "<id>:<phase>" to a shared log (to assert cross-worker ordering), and
can be told to fail in a given phase."""
from __future__ import annotations

import collections
from typing import Any, Dict, Iterable, List, Optional

from ..common import datatypes
from . import abstract_worker

WorkerState = datatypes.WorkerState


class MockWorker(abstract_worker.Worker):
  def __init__(self, worker_id: str, roles: Iterable[str], resources: Optional[Dict[str, Any]] = None,
               log: Optional[List[str]] = None, fail_stop: bool = False, fail_in: Iterable[str] = ()):
    self._info = datatypes.WorkerInfo(worker_id=worker_id, roles=frozenset(roles), resources=resources or {})
    self.call_counts: collections.Counter = collections.Counter()
    self._log = log
    self._fail_in = set(fail_in) | ({"stop"} if fail_stop else set())

  def _enter(self, phase: str, state: WorkerState) -> datatypes.Response:
    self.call_counts[phase] += 1
    self.state = state
    if self._log is not None:
      self._log.append(f"{self._info.worker_id}:{phase}")
    if phase in self._fail_in:
      verb = "refused to stop" if phase == "stop" else f"failed in {phase}"
      raise RuntimeError(f"{self._info.worker_id} {verb}")
    return datatypes.Response()

  def info(self) -> datatypes.WorkerInfo:
    return self._info

  def heartbeat(self) -> datatypes.HealthReport:
    return datatypes.HealthReport(state=self.state)

  def initialize(self) -> datatypes.Response:
    return self._enter("initialize", WorkerState.INITIALIZING)

  def compile(self, dummy_data: Any = None) -> datatypes.Response:
    return self._enter("compile", WorkerState.READY)

  def start(self) -> datatypes.Response:
    return self._enter("start", WorkerState.READY)

  def stop(self) -> datatypes.Response:
    return self._enter("stop", WorkerState.STOPPED)
