"""Rollout worker (tunix/experimental/worker/rollout_worker.py:40-505): lifecycle around a
`RolloutManager`; `generate(requests=... | prompts=...)` is what the engine dispatches to; the
weight-sync destination phases are forwarded to the manager."""
from __future__ import annotations

import asyncio
from typing import Any, Callable, List, Optional, Sequence

from ..common import datatypes
from ..rollout import manager as manager_lib
from . import abstract_worker

WorkerState = datatypes.WorkerState


class RolloutWorker(abstract_worker.Worker):
  def __init__(self, manager_factory: Callable[[], manager_lib.RolloutManager], *, worker_id: str = "rollout_worker"):
    self._factory, self._worker_id = manager_factory, worker_id
    self._manager: Optional[manager_lib.RolloutManager] = None
    self._state = WorkerState.PENDING
    self._inflight = 0
    self._last_error: Optional[str] = None
    self._seq = 0

  @property
  def manager(self) -> manager_lib.RolloutManager:
    if self._manager is None:
      self._manager = self._factory()
    return self._manager

  def _version(self) -> int:
    return int(getattr(self.manager.sampler, "policy_version", 0))

  def initialize(self) -> datatypes.Response:
    with self._phase(WorkerState.INITIALIZING):
      self.manager.sampler.initialize()
    return datatypes.Response(metadata={"worker_id": self._worker_id})

  def compile(self, dummy_data: Any = None) -> datatypes.Response:
    with self._phase(WorkerState.COMPILING):
      pass                                   # CUDA graphs are captured on first use per batch bucket
    return datatypes.Response()

  def start(self) -> datatypes.Response:
    if self.state != WorkerState.READY:
      raise RuntimeError(f"Cannot start RolloutWorker from {self.state.value}.")
    return datatypes.Response()

  def stop(self) -> datatypes.Response:
    if self.state == WorkerState.READY:
      self.state = WorkerState.DRAINING
    self._state = WorkerState.STOPPED
    return datatypes.Response()

  def info(self) -> datatypes.WorkerInfo:
    return datatypes.WorkerInfo(worker_id=self._worker_id, roles=frozenset({"rollout"}),
                                resources={"sampler": type(self.manager.sampler).__name__})

  def heartbeat(self) -> datatypes.HealthReport:
    return datatypes.HealthReport(state=self.state, inflight=self._inflight, policy_version=self._version(),
                                  last_error=self._last_error)

  async def generate(self, requests: Optional[Sequence[datatypes.RolloutRequest]] = None,
                     prompts: Optional[Sequence[Any]] = None, **generation_kwargs) -> List[datatypes.RolloutResponse]:
    if self.state not in (WorkerState.READY, WorkerState.SYNCING):
      raise RuntimeError(f"RolloutWorker is not ready: {self.state.value}.")
    reqs = list(requests or [])
    for p in prompts or []:
      self._seq += 1
      reqs.append(datatypes.RolloutRequest(request_id=f"{self._worker_id}_{self._seq}", prompt=p,
                                           prompt_id=f"{self._worker_id}_{self._seq}",
                                           generation_kwargs=dict(generation_kwargs)))
    self._inflight += len(reqs)
    try:
      return await self.manager.generate(reqs)
    except Exception as e:
      self._last_error = str(e)
      raise
    finally:
      self._inflight -= len(reqs)

  # ---- weight-sync destination ---------------------------------------------------------------
  async def bind_weight_sync(self, **kw):
    return await self.manager.bind_weight_sync(**kw)

  async def get_weight_sync_metadata(self, **kw):
    return await self.manager.get_weight_sync_metadata(**kw)

  async def get_weight_sync_status(self, **kw):
    return await self.manager.get_weight_sync_status(**kw)

  async def pre_weight_sync(self, sync_request: Any = None, **kw):
    if self.state == WorkerState.READY:
      self.state = WorkerState.SYNCING
    return await self.manager.pre_weight_sync(sync_request, **kw)

  async def weight_sync(self, sync_request: Any = None, **kw):
    return await self.manager.weight_sync(sync_request, **kw)

  async def post_weight_sync(self, sync_request: Any = None, **kw):
    out = await self.manager.post_weight_sync(sync_request, **kw)
    if self.state == WorkerState.SYNCING:
      self.state = WorkerState.READY
    return out

  async def abort_weight_sync(self, sync_request: Any = None, **kw):
    out = await self.manager.abort_weight_sync(sync_request, **kw)
    if self.state == WorkerState.SYNCING:
      self.state = WorkerState.READY
    return out
