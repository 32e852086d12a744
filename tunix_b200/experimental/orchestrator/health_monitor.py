"""Heartbeat polling with per-state deadlines (tunix/experimental/orchestrator/health_monitor.py:35-167).
Transient states have a time limit (COMPILING 30 min, SYNCING 10 min, DRAINING 5 min); a worker
that stays longer is reported as overdue so the orchestrator can fence or fail it. Steady states
have no limit. The clock is injectable, so the policy is tested without sleeping; a heartbeat
that raises is recorded as an ERROR report instead of breaking the poll."""
from __future__ import annotations

import concurrent.futures
import dataclasses
import logging
import time
from typing import Callable, Dict, List, Optional, Tuple

from ..common import datatypes
from . import worker_registry

WorkerState = datatypes.WorkerState
DEFAULT_STATE_DEADLINES_S: Dict[WorkerState, float] = {
    WorkerState.COMPILING: 30 * 60.0, WorkerState.SYNCING: 10 * 60.0, WorkerState.DRAINING: 5 * 60.0}


@dataclasses.dataclass(kw_only=True)
class OverdueWorker:
  worker_id: str
  state: str
  elapsed_s: float
  deadline_s: float


class HealthMonitor:
  def __init__(self, registry: worker_registry.WorkerRegistry, *,
               state_deadlines_s: Optional[Dict[WorkerState, float]] = None,
               clock: Callable[[], float] = time.monotonic, max_workers: int = 32,
               executor: Optional[concurrent.futures.ThreadPoolExecutor] = None,
               heartbeat_timeout_s: Optional[float] = None):
    self._registry = registry
    self._deadlines = dict(DEFAULT_STATE_DEADLINES_S if state_deadlines_s is None else state_deadlines_s)
    self._clock = clock
    self._since: Dict[str, Tuple[WorkerState, float]] = {}
    self._owns = executor is None
    self._executor = executor or concurrent.futures.ThreadPoolExecutor(max_workers=max_workers)
    self._hb_timeout = heartbeat_timeout_s

  def close(self) -> None:
    if self._owns:
      self._executor.shutdown(wait=True)

  def __enter__(self):
    return self

  def __exit__(self, *exc):
    self.close()
    return False

  def poll(self) -> Dict[str, datatypes.HealthReport]:
    ids = self._registry.worker_ids()

    def one(wid: str):
      try:
        worker = self._registry.get(wid)
      except KeyError:
        return wid, None
      try:
        return wid, worker.heartbeat()
      except Exception as e:      # a dead worker must show up in the report, not abort the poll
        return wid, datatypes.HealthReport(state=WorkerState.ERROR, last_error=f"heartbeat failed: {e!r}")
    futs = {self._executor.submit(one, wid): wid for wid in ids}
    reports: Dict[str, datatypes.HealthReport] = {}
    done, pending = concurrent.futures.wait(futs, timeout=self._hb_timeout)
    for f in done:
      wid, rep = f.result()
      if rep is not None:
        reports[wid] = rep
    for f in pending:             # no answer within the heartbeat timeout
      f.cancel()
      reports[futs[f]] = datatypes.HealthReport(state=WorkerState.ERROR, last_error="heartbeat timed out")
    now = self._clock()
    for wid, rep in reports.items():
      prev = self._since.get(wid)
      if prev is None or prev[0] != rep.state:
        self._since[wid] = (rep.state, now)
    for wid in set(self._since) - set(ids):
      del self._since[wid]
    return reports

  def overdue(self) -> List[OverdueWorker]:
    now = self._clock()
    out = []
    for wid, (state, since) in sorted(self._since.items()):
      limit = self._deadlines.get(state)
      if limit is not None and now - since > limit:
        out.append(OverdueWorker(worker_id=wid, state=getattr(state, "value", str(state)), elapsed_s=now - since,
                                 deadline_s=limit))
    return out

  def unhealthy(self) -> List[str]:
    """Workers whose last report was ERROR (including failed or timed-out heartbeats)."""
    return sorted(w for w, (s, _) in self._since.items() if s == WorkerState.ERROR)
