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
import threading
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


class _DispatchWindow:
  """Back-pressure between dispatch and training: prompt number i may be dispatched once
  i < (policy_version + max_staleness + 1) * mini_batch_size, i.e. rollouts never run more than `max_staleness`
  optimizer steps ahead of the policy that will train on them. The trainer calls `advance()` after every step;
  the dispatcher sleeps on a condition in between (no polling)."""

  def __init__(self, per_step: int, max_staleness: Optional[int]):
    self.per_step, self.max_staleness = per_step, max_staleness
    self.version = 0
    self._moved = asyncio.Condition()

  def _open_for(self, index: int) -> bool:
    return self.max_staleness is None or index < (self.version + self.max_staleness + 1) * self.per_step

  async def admit(self, index: int) -> None:
    if self._open_for(index):
      return
    async with self._moved:
      await self._moved.wait_for(lambda: self._open_for(index))

  async def advance(self, version: int) -> None:
    async with self._moved:
      self.version = version
      self._moved.notify_all()


@dataclasses.dataclass
class _StepLedger:
  """What one optimizer step consumed."""
  groups: List[List[Any]] = dataclasses.field(default_factory=list)
  rewards: List[float] = dataclasses.field(default_factory=list)
  micro_batches: int = 0
  train_result: Any = None

  def summary(self, step: int, version: int) -> RLStepResult:
    r = np.asarray(self.rewards, dtype=np.float64)
    return RLStepResult(step=step, policy_version=version, num_rollouts=len(self.rewards),
                        num_microbatches=self.micro_batches, reward_mean=float(r.mean()) if r.size else 0.0,
                        reward_std=float(r.std()) if r.size else 0.0, train_result=self.train_result)


def _as_prompt_item(item: Any, index: int) -> Any:
  """Every dispatched prompt needs an id; plain prompts and dicts without one get `prompt_<index>`."""
  if isinstance(item, dict):
    return {"prompt_id": f"prompt_{index}", **item}
  if hasattr(item, "prompt_id"):
    return item
  return {"prompt": item, "prompt_id": f"prompt_{index}"}


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
    self._window: Optional[_DispatchWindow] = None        # made inside the running loop
    self._expected = self._received = 0                   # rollouts asked for / come back
    self._dispatch_done = False

  # ---- stage 1: dispatch
  async def rollout_dispatch_stage(self, engine, train_dataset=None) -> None:
    source = train_dataset if train_dataset is not None else self.dataset
    if source is None:
      raise ValueError("StandardRLProgram requires a dataset either at init or in run().")
    window = self._window or _DispatchWindow(self.mini_batch_size, self.max_staleness)
    for index, item in enumerate(source):
      await window.admit(index)
      await engine.dispatch_rollouts([_as_prompt_item(item, index)], group_size=self.group_size,
                                     policy_version=self.policy_version)
      self._expected += self.group_size
    self._dispatch_done = True
    await self._close_intake_if_complete()

  async def _close_intake_if_complete(self) -> None:
    """The data has run out once every prompt is dispatched and every rollout asked for has come back: the
    grouping queue then drains (complete groups still go out, nothing new comes in), which ends the critic, whose
    exit drains the scored queue, which lets the trainer finish its last - possibly shorter - step and stop. A
    rollout that never comes back keeps the program waiting; engines bound their rollouts, this program does not."""
    if self._dispatch_done and self._received >= self._expected:
      await self.raw_q.prepare_clear()

  # ---- stage 2: collect finished rollouts
  async def polling_stage(self, engine) -> None:
    while True:
      try:
        finished = await engine.poll_rollouts(timeout_s=0.2)
      except asyncio.CancelledError:
        return
      except Exception as e:       # noqa: BLE001 - a flaky worker must not end the collection
        logging.warning("Error in polling_stage: %s", e)
        await asyncio.sleep(0.01)
        continue
      for item in finished or []:
        await self.raw_q.put(item)
        self._received += 1
      if finished:
        await self._close_intake_if_complete()

  # ---- stage 3: score complete groups
  def _score(self, item: Any) -> float:
    if self.reward_fns:
      return float(sum(fn(item) for fn in self.reward_fns))
    return float(getattr(item.traj, "reward", 0.0))

  async def critique_stage(self, engine) -> None:
    while True:
      try:
        group = await self.raw_q.get_group()
      except asyncio.CancelledError:
        return
      if not group:
        await self.scored_q.prepare_clear()      # nothing more will be scored
        return
      rewards = [self._score(item) for item in group]
      payloads = self.algo.create_trainer_payloads(group, rewards=rewards)
      group_id = getattr(group[0], "group_id", "default")
      for index, (source, payload, reward) in enumerate(zip(group, payloads, rewards)):
        scored = datatypes.TrajectoryItem(pair_index=index, group_id=group_id, start_step=0,
                                          traj=datatypes.Trajectory(reward=reward),
                                          policy_version=getattr(source, "policy_version", 0))
        scored.payload = payload
        await self.scored_q.put(scored)

  # ---- stage 4: train
  async def _micro_batches(self, engine, items: List[Any]) -> List[Any]:
    """One group's payloads packed into micro-batches, with reference log-probs when the algorithm has a KL term."""
    batches = self.assembler.pack([item.payload for item in items])
    if not getattr(self.algo, "requires_reference_kl", False):
      return batches
    with_ref = []
    for batch in batches:
      if not isinstance(batch, rl_common.TrainExample):
        raise TypeError("Reference KL requires an assembler that returns rl_common.TrainExample microbatches; "
                        f"got {type(batch).__name__}.")
      ref_logps = await engine.per_token_logps(datatypes.Role.REFERENCE, items=batch)
      with_ref.append(batch_assembly.with_ref_per_token_logps(batch, ref_logps))
    return with_ref

  async def _one_step(self, engine) -> _StepLedger:
    """Accumulates gradients over up to `mini_batch_size` groups and applies the optimizer with the very last
    micro-batch of the step. A group is trained on as soon as it is scored - only its last micro-batch waits
    until the next group has arrived (or the queue has drained), because that decides whether it closes the
    step: when the data runs out mid-step the groups that did arrive still get their update."""
    ledger = _StepLedger()
    items = await self.scored_q.get_batch(num_groups=1)
    position = 0
    while items:
      ledger.groups.append(items)
      ledger.rewards.extend(float(getattr(item.traj, "reward", 0.0)) for item in items)
      batches = await self._micro_batches(engine, items)
      ledger.micro_batches += len(batches)
      for batch in batches[:-1]:
        ledger.train_result = await engine.train_step(batch, role=datatypes.Role.ACTOR, accumulate_gradients=True,
                                                      apply_optimizer=False)
      last_slot = position == self.mini_batch_size - 1
      upcoming = [] if last_slot else await self.scored_q.get_batch(num_groups=1)
      if batches:
        ledger.train_result = await engine.train_step(batches[-1], role=datatypes.Role.ACTOR,
                                                      accumulate_gradients=True, apply_optimizer=not upcoming)
      items, position = upcoming, position + 1
    return ledger

  async def train_stage(self, engine, num_steps: Optional[int] = None) -> None:
    step = 0
    while num_steps is None or step < num_steps:
      if self.on_step_begin:
        self.on_step_begin(self.step)
      ledger = await self._one_step(engine)
      if not ledger.groups:
        return
      published = (await engine.sync_weights(role=datatypes.Role.ACTOR)) if self.sync_weights else None
      self.policy_version = published or self.step + 1
      if self._window is not None:
        await self._window.advance(self.policy_version)
      self.scored_q.commit(step, groups=ledger.groups)
      self.last_step_result = ledger.summary(step, self.policy_version)
      self.history.append(self.last_step_result)
      if self.on_step_end:
        self.on_step_end(step, self.last_step_result)
      step += 1

  # ---- supervision
  async def run_async(self, engine, train_dataset=None, num_steps: Optional[int] = None, **kwargs) -> None:
    """Runs the four stages until the trainer has done `num_steps` (or the data ran out). A failure of the
    dispatcher or the critic cancels training and is re-raised; the poller only logs."""
    self._is_running = True
    await self.raw_q.clear()                     # a program can be run again: queues and counters start over
    await self.scored_q.clear()
    self._expected = self._received = 0
    self._dispatch_done = False
    self._window = _DispatchWindow(self.mini_batch_size, self.max_staleness)
    self._window.version = self.policy_version
    dispatch = asyncio.create_task(self.rollout_dispatch_stage(engine, train_dataset))
    poll = asyncio.create_task(self.polling_stage(engine))
    critique = asyncio.create_task(self.critique_stage(engine))
    train = asyncio.create_task(self.train_stage(engine, num_steps))
    watched = {train, dispatch, critique}
    try:
      while not train.done():
        finished, _ = await asyncio.wait(watched, return_when=asyncio.FIRST_COMPLETED)
        watched -= finished
        broken = next((t for t in finished if t is not train and not t.cancelled() and t.exception()), None)
        if broken is not None:
          train.cancel()
          raise broken.exception()
      await train
    finally:
      self._is_running = False
      await self.raw_q.prepare_clear()
      await self.scored_q.prepare_clear()
      helpers = [dispatch, poll, critique]
      for task in helpers:
        task.cancel()
      await asyncio.gather(*helpers, return_exceptions=True)

  def run(self, engine, train_dataset=None, num_steps: Optional[int] = None, **kwargs) -> None:
    """Synchronous entry point. Called where an event loop is already running (a notebook, a coroutine of the
    caller), the program gets a loop of its own on another thread and the caller blocks until it is done."""
    try:
      asyncio.get_running_loop()
    except RuntimeError:
      asyncio.run(self.run_async(engine, train_dataset, num_steps, **kwargs))
      return
    failure: List[BaseException] = []

    def own_loop():
      try:
        asyncio.run(self.run_async(engine, train_dataset, num_steps, **kwargs))
      except BaseException as e:  # noqa: BLE001 - re-raised in the caller's thread
        failure.append(e)
    worker = threading.Thread(target=own_loop, name="rl-program")
    worker.start()
    worker.join()
    if failure:
      raise failure[0]
