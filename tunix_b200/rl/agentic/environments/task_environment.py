"""Single-turn environment: the first action ends the episode and is scored by the reward function
(tunix/rl/agentic/environments/task_environment.py:29-117)."""
from __future__ import annotations

import logging
from typing import Any, Dict

from ..agents import agent_types
from . import base_environment

_PASSED_BY_LEARNER = ("reward_fn", "group_id")


class TaskEnvironment(base_environment.BaseTaskEnv):

  def __init__(self, single_example: Dict[str, Any] = None, *, reward_fn=None, **kwargs):
    if reward_fn is None:
      logging.warning("No reward_fn provided.")
    super().__init__(task=single_example, reward_fn=reward_fn, max_steps=1, **kwargs)

  def _initial_observation(self) -> Dict[str, Any]:
    return self.task

  def _step_impl(self, action: Any) -> base_environment.EnvStepResult:
    return self.final(action.action if isinstance(action, agent_types.Action) else action)

  @classmethod
  def from_dict(cls, env_args: Dict[str, Any]) -> "TaskEnvironment":
    """`env_args` is the task record itself, with the learner's extras mixed in under reserved keys."""
    extras = {k: env_args.get(k) for k in _PASSED_BY_LEARNER}
    record = {k: v for k, v in env_args.items() if k not in _PASSED_BY_LEARNER}
    return cls(single_example=record, **extras)
