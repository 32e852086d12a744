"""The RL loop as four concurrent stages over an engine
(tunix/experimental/orchestrator/rl_program.py:39-384):

  dispatch  - expands every prompt into `group_size` rollout requests, with back-pressure so
              that rollouts never run more than `max_staleness` policy versions ahead;
  polling   - long-polls finished rollouts into a grouping queue (stale items are dropped);
  critique  - scores a complete group (reward functions or the environment's reward) and turns
              it into per-trajectory trainer payloads with group-relative advantages;
  train     - per step: `mini_batch_size` groups, assembled into micro-batches (reference
              log-probs added when the algorithm needs KL), gradients accumulated over all of
              them, one optimizer update on the last, then a weight-sync round.
"""
from __future__ import annotations

import abc
import asyncio
import dataclasses
import logging
from typing import Any, Callable, Iterable, List, Optional, Sequence

import numpy as np

from ...rl import common as rl_common
from ..common import datatypes
from ..queue_manager import trajectory_queue_manager as tqm
from . import algorithm_adapter, batch_assembly, rl_engine_interface


@dataclasses.dataclass
class RLStepResult:
  step: int
  policy_version: int
  num_rollouts: int
  num_microbatches: int
  reward_mean: float
  reward_std: float
  train_result: Any = None


class RLProgram(abc.ABC):
  def __init__(self):
    self._is_running = False
    self.policy_version = 0
    self.last_step_result: Optional[RLStepResult] = None

  @property
  def step(self) -> int:
    return self.policy_version

  @abc.abstractmethod
  def run(self, engine: rl_engine_interface.AbstractRLEngine, train_dataset: Optional[Iterable[Any]] = None,
          num_steps: Optional[int] = None, **kwargs: Any) -> None: ...


class StandardRLProgram(RLProgram):
  def __init__(self, algo: algorithm_adapter.AlgorithmAdapter, dataset: Optional[Iterable[Any]] = None,
               reward_fns: Optional[Sequence[Callable[..., Any]]] = None, assembler: Any = None, group_size: int = 8,
               mini_batch_size: int = 4, max_staleness: Optional[int] = None, sync_weights: bool = True,
               on_step_begin: Optional[Callable[[int], None]] = None,
               on_step_end: Optional[Callable[[int, Any], None]] = None):
    super().__init__()
    if max_staleness is not None and max_staleness < 0:
      raise ValueError("max_staleness must be non-negative or None.")
    self.dataset, self.algo = dataset, algo
    self.reward_fns = list(reward_fns or [])
    self.group_size = getattr(algo, "group_size", group_size)
    self.mini_batch_size = getattr(algo, "mini_batch_size", mini_batch_size)
    self.assembler = assembler or batch_assembly.SequencePackedBatchAssembler(getattr(algo, "max_packed_len", 8192))
    self.max_staleness, self.sync_weights = max_staleness, sync_weights
    self.on_step_begin, self.on_step_end = on_step_begin, on_step_end
    self.raw_q = tqm.TrajectoryQueueManager.create(group_size=self.group_size, max_staleness=max_staleness,
                                                   current_policy_version=lambda: self.policy_version)
    self.scored_q = tqm.TrajectoryQueueManager.create(group_size=self.group_size)
    self.history: List[RLStepResult] = []

  async def _wait_for_dispatch_window(self, prompt_idx: int) -> None:
    if self.max_staleness is None:
      return
    ahead = self.mini_batch_size * (self.max_staleness + 1)
    while prompt_idx - self.policy_version * self.mini_batch_size >= ahead:
      await asyncio.sleep(0.005)

  async def rollout_dispatch_stage(self, engine, train_dataset=None) -> None:
    ds = train_dataset if train_dataset is not None else self.dataset
    if ds is None:
      raise ValueError("StandardRLProgram requires a dataset either at init or in run().")
    for i, item in enumerate(ds):
      await self._wait_for_dispatch_window(i)
      if isinstance(item, dict):
        item = dict(item)
        item.setdefault("prompt_id", f"prompt_{i}")
      elif not hasattr(item, "prompt_id"):
        item = {"prompt": item, "prompt_id": f"prompt_{i}"}
      await engine.dispatch_rollouts([item], group_size=self.group_size, policy_version=self.policy_version)

  async def polling_stage(self, engine) -> None:
    while True:
      try:
        for it in await engine.poll_rollouts(timeout_s=0.2) or []:
          await self.raw_q.put(it)
      except asyncio.CancelledError:
        break
      except Exception as e:
        logging.warning("Error in polling_stage: %s", e)
        await asyncio.sleep(0.01)

  async def critique_stage(self, engine) -> None:
    while True:
      try:
        group = await self.raw_q.get_group()
      except asyncio.CancelledError:
        break
      if not group:
        break
      rewards = [float(sum(fn(it) for fn in self.reward_fns)) if self.reward_fns
                 else float(getattr(it.traj, "reward", 0.0)) for it in group]
      for idx, (payload, r) in enumerate(zip(self.algo.create_trainer_payloads(group, rewards=rewards), rewards)):
        item = datatypes.TrajectoryItem(pair_index=idx, group_id=getattr(group[0], "group_id", "default"),
                                        start_step=0, traj=datatypes.Trajectory(reward=r),
                                        policy_version=getattr(group[idx], "policy_version", 0))
        item.payload = payload
        await self.scored_q.put(item)

  async def train_stage(self, engine, num_steps: Optional[int] = None) -> None:
    step = 0
    while num_steps is None or step < num_steps:
      if self.on_step_begin:
        self.on_step_begin(self.step)
      groups, rewards, n_micro, result = [], [], 0, None
      for g in range(self.mini_batch_size):
        items = await self.scored_q.get_batch(num_groups=1)
        if not items:
          break
        groups.append(items)
        rewards += [float(getattr(i.traj, "reward", 0.0)) for i in items]
        batches = self.assembler.pack([i.payload for i in items])
        if getattr(self.algo, "requires_reference_kl", False):
          scored = []
          for b in batches:
            if not isinstance(b, rl_common.TrainExample):
              raise TypeError("Reference KL requires an assembler that returns rl_common.TrainExample microbatches; "
                              f"got {type(b).__name__}.")
            scored.append(batch_assembly.with_ref_per_token_logps(
                b, await engine.per_token_logps(datatypes.Role.REFERENCE, items=b)))
          batches = scored
        n_micro += len(batches)
        last_group = g == self.mini_batch_size - 1
        for bi, b in enumerate(batches):
          result = await engine.train_step(b, role=datatypes.Role.ACTOR, accumulate_gradients=True,
                                           apply_optimizer=last_group and bi == len(batches) - 1)
      if not groups:
        break
      if self.sync_weights:
        self.policy_version = (await engine.sync_weights(role=datatypes.Role.ACTOR)) or self.step + 1
      else:
        self.policy_version = self.step + 1
      self.scored_q.commit(step, groups=groups)
      self.last_step_result = RLStepResult(
          step=step, policy_version=self.policy_version, num_rollouts=len(rewards), num_microbatches=n_micro,
          reward_mean=float(np.mean(rewards)) if rewards else 0.0, reward_std=float(np.std(rewards)) if rewards else 0.0,
          train_result=result)
      self.history.append(self.last_step_result)
      if self.on_step_end:
        self.on_step_end(step, self.last_step_result)
      step += 1

  async def run_async(self, engine, train_dataset=None, num_steps: Optional[int] = None, **kwargs) -> None:
    self._is_running = True
    side = [asyncio.create_task(self.rollout_dispatch_stage(engine, train_dataset)),
            asyncio.create_task(self.polling_stage(engine)), asyncio.create_task(self.critique_stage(engine))]
    try:
      train = asyncio.create_task(self.train_stage(engine, num_steps))
      watch = {train, side[0], side[2]}
      while not train.done():
        done, _ = await asyncio.wait(watch, return_when=asyncio.FIRST_COMPLETED)
        for t in done:
          watch.discard(t)
          if t is not train and not t.cancelled() and t.exception() is not None:
            train.cancel()
            raise t.exception()
      await train
    finally:
      self._is_running = False
      await self.raw_q.prepare_clear()
      await self.scored_q.prepare_clear()
      for t in side:
        t.cancel()
      await asyncio.gather(*side, return_exceptions=True)

  def run(self, engine, train_dataset=None, num_steps: Optional[int] = None, **kwargs) -> None:
    asyncio.run(self.run_async(engine, train_dataset, num_steps, **kwargs))
