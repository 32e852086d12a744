"""Episode worker pool feeding a grouping queue (behaviour of
tunix/rl/agentic/pipeline/rollout_orchestrator.py:47-392; see `RolloutOrchestrator`)."""
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


class _PairSource:
  """Serialises access to a sync or async stream of (agent, env) pairs for several consumers."""

  def __init__(self, stream: Union[Iterable[Pair], AsyncIterable[Pair]]):
    self._async = hasattr(stream, "__aiter__")
    self._it = stream.__aiter__() if self._async else iter(stream)
    self._turn = asyncio.Lock()
    self.dry = False

  async def take(self) -> Optional[Pair]:
    async with self._turn:
      if self.dry:
        return None
      try:
        return await self._it.__anext__() if self._async else next(self._it)
      except (StopIteration, StopAsyncIteration):
        self.dry = True
        return None


class RolloutOrchestrator:
  """A fixed pool of `max_concurrency` episode workers over a stream of (agent, env) pairs.

  Each worker repeatedly takes the next pair, holds the rollout side of the `RolloutSyncLock` for the length
  of the episode (so a weight sync waits for running episodes and keeps new ones from starting), collects the
  trajectory and hands it to a `GroupQueueManager` under its group key. When the stream is dry and every worker
  has returned, the queue is switched to draining and `yield_batches` ends. The first failing episode poisons the
  queue - the consumer sees the error - and stops the pool; a consumer that leaves early cancels the workers.
  """

  def __init__(self, *, rollout_sync_lock: utils.RolloutSyncLock,
               engine_cls: Type[TrajectoryCollectEngine] = TrajectoryCollectEngine,
               engine_kwargs: Optional[Dict[str, Any]] = None, max_concurrency: Optional[int] = None):
    self.engine_cls = engine_cls
    self.engine_kwargs = engine_kwargs or {}
    self.max_concurrency = max_concurrency
    self._workers: List[asyncio.Task] = []
    self._halt = asyncio.Event()
    self._running = asyncio.Event()
    self._group_queue_manager: Optional[GroupQueueManager] = None
    self._rollout_sync_lock = rollout_sync_lock

  async def _collect_trajectory(self, agent, env, mode: Optional[str] = None,
                                model_call_kwargs: Optional[Dict[str, Any]] = None):
    kw = dict(self.engine_kwargs)
    if model_call_kwargs:
      kw["model_call_kwargs"] = model_call_kwargs
    engine = self.engine_cls(agent, env, **kw)
    return await (engine.collect(mode) if mode else engine.collect())

  async def _episode(self, agent, env, queue: GroupQueueManager, group_key_fn, start_step_fn, collect_mode) -> None:
    index = env.extra_kwargs["pair_index"]
    # the lock is a thread lock: wait for it off the event loop, other episodes keep running meanwhile
    await asyncio.get_running_loop().run_in_executor(None, self._rollout_sync_lock.acquire_rollout)
    try:
      traj = await self._collect_trajectory(agent, env, mode=collect_mode)
      await queue.put(TrajectoryItem(pair_index=index, group_id=group_key_fn(index, env, traj),
                                     start_step=start_step_fn() if start_step_fn else 0, traj=traj,
                                     metadata={"generation_id": index}))
    finally:
      self._rollout_sync_lock.release_rollout()

  async def _worker(self, source: _PairSource, queue: GroupQueueManager, group_key_fn, start_step_fn,
                    collect_mode) -> None:
    while not self._halt.is_set():
      pair = await source.take()
      if pair is None:
        return
      try:
        await self._episode(pair[0], pair[1], queue, group_key_fn, start_step_fn, collect_mode)
      except asyncio.CancelledError:
        raise
      except BaseException as e:
        for sub in getattr(e, "exceptions", [e]):
          logging.error("episode %s failed: %s", pair[1].extra_kwargs.get("pair_index"), sub)
        traceback.print_exc()
        await queue.put_exception(e)
        self._halt.set()
        raise

  async def run_producers_from_stream(self, pairs_stream: Union[Iterable[Pair], AsyncIterable[Pair]], *,
                                      group_size: int,
                                      group_key_fn: Callable[[int, BaseTaskEnv, Trajectory], Hashable] = lambda i, _, __: i,
                                      collect_mode: Optional[str] = None,
                                      start_step_fn: Optional[Callable[[], int]] = None) -> None:
    if not self.max_concurrency:
      raise ValueError("max_concurrency must be set to use start_producers.")
    if self._group_queue_manager:
      raise RuntimeError("Orchestrator is already running.")
    queue = self._group_queue_manager = GroupQueueManager(
        key_fn=lambda x: getattr(x, "group_id", getattr(x, "prompt_id", id(x))), group_size=group_size)
    self._halt.clear()
    source = _PairSource(pairs_stream)
    self._workers = [asyncio.create_task(self._worker(source, queue, group_key_fn, start_step_fn, collect_mode))
                     for _ in range(self.max_concurrency)]
    self._running.set()
    try:
      results = await asyncio.gather(*self._workers, return_exceptions=True)
      failed = next((r for r in results if isinstance(r, BaseException) and not isinstance(r, asyncio.CancelledError)),
                    None)
      if failed is not None:
        raise failed
    except asyncio.CancelledError:
      for w in self._workers:
        w.cancel()
      raise
    finally:
      await asyncio.shield(queue.prepare_clear())

  async def yield_batches(self, batch_size: int, start_timeout: float = 5.0):
    """Yields lists of `TrajectoryItem`. The producer coroutine is usually started with
    `create_task` right before this call and may not have run yet, so its start is awaited
    for up to `start_timeout` seconds."""
    if not self._group_queue_manager:
      try:
        await asyncio.wait_for(self._running.wait(), start_timeout)
      except asyncio.TimeoutError:
        raise RuntimeError("Producers have not been started.") from None
    try:
      while not self._halt.is_set():
        batch = await self._group_queue_manager.get_batch(batch_size)
        if not batch:
          break
        yield batch
    except (GeneratorExit, asyncio.CancelledError):
      pass
    finally:
      self._halt.set()
      for w in self._workers:
        if not w.done():
          w.cancel()
