"""Heartbeat polling with per-state deadlines (tunix/experimental/orchestrator/health_monitor.py:35-167).

Two small parts:

  * `DwellTracker` remembers, per worker, which state it was last seen in and since when (on an injectable
    clock). Transient states carry a time limit (COMPILING 30 min, SYNCING 10 min, DRAINING 5 min); a worker that
    dwells longer is *overdue*, so the orchestrator can fence or fail it. Steady states have no limit.
  * `HealthMonitor.poll()` asks every registered worker for a heartbeat in parallel. A heartbeat that raises, or
    that does not answer within `heartbeat_timeout_s`, becomes an ERROR report - a dead worker must show up in the
    result, not abort the poll. Workers that left the registry are forgotten.

Nothing here sleeps or spawns a timer: the orchestrator decides when to poll, and tests drive the clock.
"""
from __future__ import annotations

import concurrent.futures
import dataclasses
import time
from typing import Callable, Dict, Iterable, List, Optional

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


@dataclasses.dataclass
class _Dwell:
  state: WorkerState
  since: float


class DwellTracker:
  """State residence times of a set of workers."""

  def __init__(self, limits: Dict[WorkerState, float], clock: Callable[[], float]):
    self.limits, self.clock = dict(limits), clock
    self._seen: Dict[str, _Dwell] = {}

  def observe(self, states: Dict[str, WorkerState], alive: Iterable[str]) -> None:
    """Records one round of observations; workers not in `alive` are dropped."""
    now = self.clock()
    for wid, state in states.items():
      known = self._seen.get(wid)
      if known is None or known.state != state:
        self._seen[wid] = _Dwell(state, now)
    for gone in set(self._seen) - set(alive):
      del self._seen[gone]

  def overdue(self) -> List[OverdueWorker]:
    now = self.clock()
    late = []
    for wid in sorted(self._seen):
      d = self._seen[wid]
      limit = self.limits.get(d.state)
      if limit is not None and now - d.since > limit:
        late.append(OverdueWorker(worker_id=wid, state=getattr(d.state, "value", str(d.state)),
                                  elapsed_s=now - d.since, deadline_s=limit))
    return late

  def in_state(self, state: WorkerState) -> List[str]:
    return sorted(wid for wid, d in self._seen.items() if d.state == state)


def _error_report(why: str) -> datatypes.HealthReport:
  return datatypes.HealthReport(state=WorkerState.ERROR, last_error=why)


class HealthMonitor:

  def __init__(self, registry: worker_registry.WorkerRegistry, *,
               state_deadlines_s: Optional[Dict[WorkerState, float]] = None,
               clock: Callable[[], float] = time.monotonic, max_workers: int = 32,
               executor: Optional[concurrent.futures.ThreadPoolExecutor] = None,
               heartbeat_timeout_s: Optional[float] = None):
    self._registry = registry
    self._dwell = DwellTracker(DEFAULT_STATE_DEADLINES_S if state_deadlines_s is None else state_deadlines_s, clock)
    self._pool = executor or concurrent.futures.ThreadPoolExecutor(max_workers=max_workers)
    self._own_pool = executor is None
    self._hb_timeout = heartbeat_timeout_s

  # ---- lifetime
  def close(self) -> None:
    if self._own_pool:
      self._pool.shutdown(wait=True)

  def __enter__(self):
    return self

  def __exit__(self, *exc):
    self.close()
    return False

  # ---- polling
  def _heartbeat(self, wid: str) -> Optional[datatypes.HealthReport]:
    try:
      worker = self._registry.get(wid)
    except KeyError:                    # unregistered between listing and asking
      return None
    try:
      return worker.heartbeat()
    except Exception as e:              # noqa: BLE001
      return _error_report(f"heartbeat failed: {e!r}")

  def poll(self) -> Dict[str, datatypes.HealthReport]:
    ids = self._registry.worker_ids()
    asked = {wid: self._pool.submit(self._heartbeat, wid) for wid in ids}
    concurrent.futures.wait(asked.values(), timeout=self._hb_timeout)
    reports: Dict[str, datatypes.HealthReport] = {}
    for wid, fut in asked.items():
      if not fut.done():                # no answer within the heartbeat timeout
        fut.cancel()
        reports[wid] = _error_report("heartbeat timed out")
      elif fut.result() is not None:
        reports[wid] = fut.result()
    self._dwell.observe({wid: rep.state for wid, rep in reports.items()}, alive=ids)
    return reports

  # ---- verdicts
  def overdue(self) -> List[OverdueWorker]:
    return self._dwell.overdue()

  def unhealthy(self) -> List[str]:
    """Workers whose last report was ERROR (including failed or timed-out heartbeats)."""
    return self._dwell.in_state(WorkerState.ERROR)
