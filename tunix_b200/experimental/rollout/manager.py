"""Concurrency core of a rollout worker (tunix/experimental/rollout/manager.py:31-317): fans
requests out to per-trajectory collectors under a concurrency cap, streams results as they
complete, gates admission through the `TrafficController` during weight syncs, and forwards
the destination-side weight-sync phases to its sampler."""
from __future__ import annotations

import asyncio
from typing import Any, Callable, Dict, List, Optional, Sequence, Union

from ..common import datatypes
from ..worker import traffic_controller as tc_lib
from . import collector as collector_lib, sampler as sampler_lib


class RolloutManager:
  def __init__(self, config: Any = None, sampler: Optional[sampler_lib.Sampler] = None, env_pool: Any = None,
               agent_factory: Optional[Callable[[], Any]] = None, max_concurrency: int = 64, tokenizer: Any = None,
               chat_parser: Any = None, drain_timeout_s: float = 300.0, env_factory: Optional[Callable[..., Any]] = None):
    if sampler is None:
      raise ValueError("RolloutManager needs a sampler (e.g. rollout.native_sampler_adapter.NativeSamplerAdapter)")
    if not isinstance(sampler, sampler_lib.Sampler):
      raise TypeError(f"Expected object implementing Sampler Protocol, got {type(sampler)}")
    self.config, self.sampler, self.env_pool = config, sampler, env_pool
    self.agent_factory, self.env_factory = agent_factory, env_factory
    self.max_concurrency, self.tokenizer, self.chat_parser = max_concurrency, tokenizer, chat_parser
    self._collectors: Dict[str, collector_lib.TrajectoryCollectorEngine] = {}
    self._tasks: Dict[str, asyncio.Task] = {}
    self._completed: asyncio.Queue = asyncio.Queue()
    self._traffic_inst: Optional[tc_lib.TrafficController] = None
    self._sem: Optional[asyncio.Semaphore] = None
    self._drain_timeout_s = drain_timeout_s

  @property
  def _traffic(self) -> tc_lib.TrafficController:
    if self._traffic_inst is None:
      self._traffic_inst = tc_lib.TrafficController()
    return self._traffic_inst

  def _env_for(self, request: datatypes.RolloutRequest):
    cfg = request.metadata.get("env_config")
    if self.env_factory is not None:
      return self.env_factory(request, cfg)
    if self.env_pool is not None and hasattr(self.env_pool, "acquire_env"):
      return self.env_pool.acquire_env(cfg)
    return None

  async def _generate_one(self, request: datatypes.RolloutRequest, on_complete=None) -> datatypes.RolloutResponse:
    if not self._traffic.is_admission_open():
      raise tc_lib.AdmissionClosedError("rollout admission is closed during weight sync")
    if self._sem is None:
      self._sem = asyncio.Semaphore(self.max_concurrency)
    col = collector_lib.TrajectoryCollectorEngine(
        request.traj_id, request, self.sampler, env_client=self._env_for(request),
        agent=self.agent_factory() if callable(self.agent_factory) else None, tokenizer=self.tokenizer,
        chat_parser=self.chat_parser)
    self._collectors[request.traj_id] = col

    async def run():
      async with self._sem:
        return await col.run()
    task = asyncio.create_task(run())
    self._tasks[request.traj_id] = task
    self._traffic.track(task)
    try:
      res = await task
    except asyncio.CancelledError:
      res = datatypes.RolloutResponse(request_id=request.request_id, prompt_id=request.prompt_id, status="CANCELLED",
                                      metadata=dict(request.metadata),
                                      error=datatypes.ErrorInfo(error_type="Cancelled", message="cancelled", retryable=True))
    finally:
      self._collectors.pop(request.traj_id, None)
      self._tasks.pop(request.traj_id, None)
    if on_complete:
      on_complete(res)
    await self._completed.put(res)
    return res

  async def generate(self, requests, on_complete=None):
    if isinstance(requests, (list, tuple)):
      return list(await asyncio.gather(*[self._generate_one(r, on_complete) for r in requests]))
    return await self._generate_one(requests, on_complete)

  async def pop_next_completed(self):
    return await self._completed.get()

  async def as_completed_stream(self, n: int):
    for _ in range(n):
      yield await self._completed.get()

  async def migrate_straggler(self, traj_id: str, target: Any = None):
    col = self._collectors.get(traj_id)
    if col is None:
      return {"migrated": False, "reason": "unknown trajectory"}
    return {"migrated": True, **(await self.sampler.migrate_kv_cache(target=target) or {})}

  def pause_all(self) -> None:
    self._traffic.transition_to_syncing()

  def resume_all(self) -> None:
    self._traffic.reopen()

  def reopen_admission(self) -> bool:
    return self._traffic.reopen()

  def cancel_all(self) -> List[asyncio.Task]:
    return self._traffic.stop_and_cancel_all()

  # destination side of a weight-sync round: gate, drain, then the sampler's own phases
  async def bind_weight_sync(self, **kw):
    return await self.sampler.bind_weight_sync(**kw)

  async def get_weight_sync_metadata(self, **kw):
    return await self.sampler.get_weight_sync_metadata(**kw)

  async def get_weight_sync_status(self, **kw):
    return await self.sampler.get_weight_sync_status(**kw)

  async def pre_weight_sync(self, sync_request: Any = None, **kw):
    self._traffic.transition_to_syncing()
    await self._traffic.drain(self._drain_timeout_s)
    for t in self._traffic.get_active_tasks():     # stragglers past the drain deadline
      t.cancel()
    return await self.sampler.pre_weight_sync(sync_request, **kw)

  async def weight_sync(self, sync_request: Any = None, **kw):
    return await self.sampler.weight_sync(sync_request, **kw)

  async def post_weight_sync(self, sync_request: Any = None, **kw):
    out = await self.sampler.post_weight_sync(sync_request, **kw)
    self._traffic.reopen()
    return out

  async def abort_weight_sync(self, sync_request: Any = None, **kw):
    out = await self.sampler.abort_weight_sync(sync_request, **kw)
    self._traffic.reopen()
    return out
