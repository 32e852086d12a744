"""Phase-by-phase bring-up and best-effort shutdown (tunix/experimental/orchestrator/lifecycle.py:28-98).
A phase (initialize, compile, start) runs on all workers in parallel and must finish everywhere
before the next begins; failures of a phase are collected and raised together. Shutdown calls
`stop()` on every worker even when earlier ones raised."""
from __future__ import annotations

import concurrent.futures
import logging
from typing import Any, Callable, List, Tuple

from . import worker_registry


class LifecycleError(RuntimeError):
  def __init__(self, phase: str, failures: List[Tuple[str, BaseException]]):
    self.phase, self.failures = phase, failures
    detail = "; ".join(f"{wid}: {err!r}" for wid, err in failures)
    super().__init__(f"{phase} failed for {len(failures)} worker(s): {detail}")


class LifecycleDriver:
  def __init__(self, registry: worker_registry.WorkerRegistry, max_workers: int = 32):
    self._registry, self._max_workers = registry, max_workers

  def _run_phase(self, phase: str, call: Callable[[Any], Any]) -> None:
    ids = self._registry.worker_ids()
    if not ids:
      return
    failures: List[Tuple[str, BaseException]] = []

    def one(wid: str):
      try:
        worker = self._registry.get(wid)
      except KeyError:
        logging.warning("Worker %r unregistered concurrently, skipping %s.", wid, phase)
        return
      call(worker)
    with concurrent.futures.ThreadPoolExecutor(max_workers=self._max_workers) as pool:
      futs = {pool.submit(one, wid): wid for wid in ids}
      for f in concurrent.futures.as_completed(futs):
        try:
          f.result()
        except Exception as e:
          failures.append((futs[f], e))
    if failures:
      raise LifecycleError(phase, sorted(failures, key=lambda t: t[0]))

  def bring_up(self, dummy_data: Any = None) -> None:
    self._run_phase("initialize", lambda w: w.initialize())
    self._run_phase("compile", lambda w: w.compile(dummy_data))
    self._run_phase("start", lambda w: w.start())

  def shutdown(self) -> None:
    self._run_phase("shutdown", lambda w: w.stop())
