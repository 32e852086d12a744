"""Environment contract of the agentic stack (tunix/rl/agentic/environments/base_environment.py:30-345).

Two levels:

  * `BaseEnv` - the gym-like surface the trajectory collector drives: `reset() -> (observation, info)`,
    `step(action) -> (observation, reward, done, info)`, `step_async`, `close`, `from_dict`. Environments are
    context managers (`with Env(...) as env:` closes them).
  * `BaseTaskEnv` - an episode over one task record with a turn budget. Subclasses say what the first
    observation is and what one turn does (`_initial_observation`, `_step_impl`) in terms of two result
    builders: `self.turn(observation)` for an intermediate step and `self.final(answer)` for the step that ends
    the episode and is scored by `reward_fn(task=..., action=...)`. Counting turns and cutting the episode at
    `max_steps` happen here, once.
"""
from __future__ import annotations

import abc
import asyncio
import dataclasses
from typing import Any, Callable, Dict, Optional, Tuple

StepTuple = Tuple[Any, float, bool, Dict[str, Any]]


@dataclasses.dataclass
class EnvStepResult:
  observation: Any
  reward: float
  done: bool
  info: Dict[str, Any]

  def as_tuple(self, force_done: bool = False) -> StepTuple:
    return self.observation, self.reward, self.done or force_done, self.info


class BaseEnv(abc.ABC):
  idx: Any = None            # position of the environment in its batch; set by whoever builds the batch

  @abc.abstractmethod
  def reset(self) -> Tuple[Dict[str, Any], Dict[str, Any]]:
    """Starts an episode: (first observation, info)."""

  @abc.abstractmethod
  def step(self, action: Any) -> StepTuple:
    """Applies an action: (next observation, reward, done, info)."""

  async def step_async(self, action: Any) -> StepTuple:
    """`step` off the event loop, so slow environments (tools, sandboxes) do not stall other episodes."""
    return await asyncio.to_thread(self.step, action)

  def close(self) -> None:
    """Releases what the environment holds. Safe to call more than once."""

  def __enter__(self):
    return self

  def __exit__(self, *exc) -> None:
    self.close()

  @classmethod
  def from_dict(cls, env_args: Dict[str, Any]) -> "BaseEnv":
    return cls(**env_args)


class BaseTaskEnv(BaseEnv):

  def __init__(self, task: Optional[Dict[str, Any]] = None, *, reward_fn: Optional[Callable[..., Any]] = None,
               max_steps: int = 1, **kwargs):
    self.task: Dict[str, Any] = task or {}
    self.reward_fn = reward_fn
    self.max_steps = max_steps
    self.step_count = 0
    self.extra_kwargs = kwargs          # e.g. group_id, pair_index set by the learner

  # ---- what a subclass provides
  def _initial_observation(self) -> Any:
    raise NotImplementedError

  def _step_impl(self, action: Any) -> EnvStepResult:
    raise NotImplementedError

  # ---- result builders for subclasses
  def score(self, answer: Any) -> float:
    return self.reward_fn(task=self.task, action=answer) if self.reward_fn is not None else 0.0

  def final(self, answer: Any, *, response: Any = None, observation: Any = None) -> EnvStepResult:
    """The step that ends the episode: `answer` is scored, `response` (default: the answer) is reported."""
    return EnvStepResult(observation={} if observation is None else observation, reward=self.score(answer), done=True,
                         info={"response": answer if response is None else response})

  def turn(self, observation: Any, *, response: Any = None, reward: float = 0.0) -> EnvStepResult:
    """An intermediate step: the episode goes on with `observation`."""
    return EnvStepResult(observation=observation, reward=reward, done=False, info={"response": response})

  # ---- the gym surface
  def reset(self) -> Tuple[Dict[str, Any], Dict[str, Any]]:
    self.step_count = 0
    return self._initial_observation(), {}

  def step(self, action: Any) -> StepTuple:
    self.step_count += 1
    return self._step_impl(action).as_tuple(force_done=self.step_count >= self.max_steps)
