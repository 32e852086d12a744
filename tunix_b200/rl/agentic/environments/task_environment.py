"""Single-turn environment: the first action ends the episode and is scored by the reward
function (tunix/rl/agentic/environments/task_environment.py:29-117)."""
from __future__ import annotations

import logging
from typing import Any, Dict

from ..agents import agent_types
from . import base_environment


class TaskEnvironment(base_environment.BaseTaskEnv):
  def __init__(self, single_example: Dict[str, Any] = None, *, reward_fn=None, **kwargs):
    if reward_fn is None:
      logging.warning("No reward_fn provided.")
    super().__init__(task=single_example, reward_fn=reward_fn, max_steps=1, **kwargs)

  def _initial_observation(self) -> Dict[str, Any]:
    return self.task

  def _step_impl(self, action: Any) -> base_environment.EnvStepResult:
    if isinstance(action, agent_types.Action):
      action = action.action
    reward = self.reward_fn(task=self.task, action=action) if self.reward_fn is not None else 0.0
    return base_environment.EnvStepResult(observation={}, reward=reward, done=True, info={"response": action})

  @classmethod
  def from_dict(cls, env_args: Dict[str, Any]) -> "TaskEnvironment":
    env_args = dict(env_args)
    reward_fn = env_args.pop("reward_fn", None)
    group_id = env_args.pop("group_id", None)
    return cls(single_example=env_args, reward_fn=reward_fn, group_id=group_id)
