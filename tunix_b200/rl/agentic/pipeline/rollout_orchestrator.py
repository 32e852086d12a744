"""Bounded-concurrency pool of episodes feeding a grouping queue
(tunix/rl/agentic/pipeline/rollout_orchestrator.py:47-392).

`run_producers_from_stream` draws (agent, env) pairs from a sync or async stream and keeps at
most `max_concurrency` episodes in flight; each episode holds the rollout side of the
`RolloutSyncLock`, so a weight sync waits for running episodes and blocks new ones. Finished
trajectories go to a `GroupQueueManager`; `yield_batches` hands out complete groups. A failing
episode poisons the queue so that the consumer sees the error; a consumer that stops early
cancels the remaining episodes.
"""
from __future__ import annotations

import asyncio
import logging
import traceback
from typing import Any, AsyncIterable, Callable, Dict, Hashable, Iterable, List, Optional, Set, Tuple, Type, Union

from ..agents.agent_types import Trajectory, TrajectoryItem
from ..agents.base_agent import ConversationAgentBase
from ..environments.base_environment import BaseTaskEnv
from ..queue_manager.group_queue_manager import GroupQueueManager
from ..trajectory.trajectory_collect_engine import TrajectoryCollectEngine
from .. import utils

Pair = Tuple[ConversationAgentBase, BaseTaskEnv]
_END = object()


class RolloutOrchestrator:
  def __init__(self, *, rollout_sync_lock: utils.RolloutSyncLock,
               engine_cls: Type[TrajectoryCollectEngine] = TrajectoryCollectEngine,
               engine_kwargs: Optional[Dict[str, Any]] = None, max_concurrency: Optional[int] = None):
    self.engine_cls = engine_cls
    self.engine_kwargs = engine_kwargs or {}
    self.max_concurrency = max_concurrency
    self._tasks: List[asyncio.Task] = []
    self._stop = asyncio.Event()
    self._started = asyncio.Event()
    self._group_queue_manager: Optional[GroupQueueManager] = None
    self._rollout_sync_lock = rollout_sync_lock

  async def _collect_trajectory(self, agent, env, mode: Optional[str] = None,
                                model_call_kwargs: Optional[Dict[str, Any]] = None):
    kw = dict(self.engine_kwargs)
    if model_call_kwargs:
      kw["model_call_kwargs"] = model_call_kwargs
    engine = self.engine_cls(agent, env, **kw)
    return await (engine.collect(mode) if mode else engine.collect())

  async def _runner(self, agent, env, manager: GroupQueueManager, group_key_fn, start_step_fn=None,
                    collect_mode: Optional[str] = None) -> int:
    """One episode under the rollout lock; its trajectory is queued with its group key."""
    pair_idx = env.extra_kwargs["pair_index"]
    loop = asyncio.get_running_loop()
    try:
      # the lock is a thread lock: take it off the event loop so waiting does not stall other episodes
      await loop.run_in_executor(None, self._rollout_sync_lock.acquire_rollout)
      try:
        traj = await self._collect_trajectory(agent, env, mode=collect_mode)
        item = TrajectoryItem(pair_index=pair_idx, group_id=group_key_fn(pair_idx, env, traj),
                              start_step=start_step_fn() if start_step_fn else 0, traj=traj,
                              metadata={"generation_id": pair_idx})
        await manager.put(item)
        return 1
      finally:
        self._rollout_sync_lock.release_rollout()
    except asyncio.CancelledError:
      raise
    except BaseException as e:
      for sub in getattr(e, "exceptions", [e]):
        logging.error("Fatal error in runner for pair %s: %s", pair_idx, sub)
      traceback.print_exc()
      await manager.put_exception(e)
      raise

  @staticmethod
  async def _next_pair(it, is_async: bool):
    try:
      return await it.__anext__() if is_async else next(it)
    except (StopIteration, StopAsyncIteration):
      return _END

  async def run_producers_from_stream(self, pairs_stream: Union[Iterable[Pair], AsyncIterable[Pair]], *,
                                      group_size: int,
                                      group_key_fn: Callable[[int, BaseTaskEnv, Trajectory], Hashable] = lambda i, _, __: i,
                                      collect_mode: Optional[str] = None,
                                      start_step_fn: Optional[Callable[[], int]] = None) -> None:
    if not self.max_concurrency:
      raise ValueError("max_concurrency must be set to use start_producers.")
    if self._group_queue_manager:
      raise RuntimeError("Orchestrator is already running.")
    manager = self._group_queue_manager = GroupQueueManager(
        key_fn=lambda x: getattr(x, "group_id", getattr(x, "prompt_id", id(x))), group_size=group_size)
    self._stop.clear()
    self._tasks.clear()
    self._started.set()
    is_async = hasattr(pairs_stream, "__aiter__")
    it = pairs_stream.__aiter__() if is_async else iter(pairs_stream)
    active: Set[asyncio.Task] = set()
    exhausted = False
    try:
      while not self._stop.is_set():
        while not exhausted and len(active) < self.max_concurrency and not self._stop.is_set():
          pair = await self._next_pair(it, is_async)
          if pair is _END:
            exhausted = True
            break
          agent, env = pair
          t = asyncio.create_task(self._runner(agent, env, manager, group_key_fn, start_step_fn, collect_mode))
          active.add(t)
          self._tasks.append(t)
        if not active:
          break
        done, active = await asyncio.wait(active, return_when=asyncio.FIRST_COMPLETED)
        for t in done:
          t.result()                    # re-raises an episode's failure
          if t in self._tasks:
            self._tasks.remove(t)
      if self._tasks:
        await asyncio.gather(*self._tasks, return_exceptions=True)
    except asyncio.CancelledError:
      raise
    except Exception as e:
      logging.error("Producer task failed: %s", e)
      await manager.put_exception(e)
      raise
    finally:
      await asyncio.shield(manager.prepare_clear())

  async def yield_batches(self, batch_size: int, start_timeout: float = 5.0):
    """Yields lists of `TrajectoryItem`. The producer coroutine is usually started with
    `create_task` right before this call and may not have run yet, so its start is awaited
    for up to `start_timeout` seconds."""
    if not self._group_queue_manager:
      try:
        await asyncio.wait_for(self._started.wait(), start_timeout)
      except asyncio.TimeoutError:
        raise RuntimeError("Producers have not been started.") from None
    try:
      while not self._stop.is_set():
        batch = await self._group_queue_manager.get_batch(batch_size)
        if not batch:
          break
        yield batch
    except (GeneratorExit, asyncio.CancelledError):
      pass
    finally:
      self._stop.set()
      for t in self._tasks:
        if not t.done():
          t.cancel()
