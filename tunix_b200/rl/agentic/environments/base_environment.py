"""Environment interfaces (tunix/rl/agentic/environments/base_environment.py:30-345).

`BaseEnv`: `reset() -> (observation, info)`, `step(action) -> (observation, reward, done, info)`,
optional `step_async`, `close`, `from_dict`. `BaseTaskEnv` adds the task dict, an optional
reward function and the step budget; subclasses implement `_initial_observation` and
`_step_impl` and get step counting and `max_steps` truncation for free.
"""
from __future__ import annotations

import abc
import asyncio
import dataclasses
from typing import Any, Callable, Dict, Optional, Tuple


@dataclasses.dataclass
class EnvStepResult:
  observation: Any
  reward: float
  done: bool
  info: Dict[str, Any]


class BaseEnv(abc.ABC):
  def __init__(self):
    self._idx = None

  @property
  def idx(self) -> Any:
    return self._idx

  @idx.setter
  def idx(self, value: Any):
    self._idx = value

  @abc.abstractmethod
  def reset(self) -> Tuple[Dict[str, Any], Dict[str, Any]]: ...

  @abc.abstractmethod
  def step(self, action: Any) -> Tuple[Any, float, bool, Dict[str, Any]]: ...

  async def step_async(self, action: Any) -> Tuple[Any, float, bool, Dict[str, Any]]:
    return await asyncio.get_event_loop().run_in_executor(None, self.step, action)

  def close(self) -> None:
    return None

  @classmethod
  def from_dict(cls, env_args: Dict[str, Any]) -> "BaseEnv":
    return cls(**env_args)


class BaseTaskEnv(BaseEnv):
  def __init__(self, task: Optional[Dict[str, Any]] = None, *, reward_fn: Optional[Callable[..., Any]] = None,
               max_steps: int = 1, **kwargs):
    super().__init__()
    self.task = task or {}
    self.reward_fn = reward_fn
    self.max_steps = max_steps
    self.step_count = 0
    self.extra_kwargs = kwargs          # e.g. group_id, pair_index set by the learner

  def _initial_observation(self) -> Any:
    raise NotImplementedError

  def _step_impl(self, action: Any) -> EnvStepResult:
    raise NotImplementedError

  def reset(self) -> Tuple[Dict[str, Any], Dict[str, Any]]:
    self.step_count = 0
    return self._initial_observation(), {}

  def step(self, action: Any) -> Tuple[Any, float, bool, Dict[str, Any]]:
    self.step_count += 1
    r = self._step_impl(action)
    return r.observation, r.reward, r.done or self.step_count >= self.max_steps, r.info

  @classmethod
  def from_dict(cls, env_args: Dict[str, Any]) -> "BaseTaskEnv":
    return cls(**env_args)
