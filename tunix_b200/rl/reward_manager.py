"""Reward managers: run the user's reward functions over (prompt, completion) pairs, sum them and
prepare per-function log metrics (tunix/rl/reward_manager.py:45-271). Reward functions receive
`prompts`, `completions`, every extra batch column as a keyword, and any algorithm-config field
whose name appears in their signature."""
from __future__ import annotations

import abc
import dataclasses
import inspect
import logging
import os
from typing import Any, Callable, Dict, List, Optional, Sequence, Union

import numpy as np

from . import algorithm_config as algo_config_lib
from . import function_registry

log = logging.getLogger(__name__)
RewardFn = Callable[..., Any]


def _calculate_scalar_reward_log_metrics(rewards: np.ndarray, prefix: str = "rewards", axis: int = 1) -> Dict[str, Any]:
  return {
      f"{prefix}/sum": (np.nansum(rewards, axis=axis), np.mean),
      f"{prefix}/mean": (np.nanmean(rewards, axis=axis), np.mean),
      f"{prefix}/min": (np.min(rewards, axis=axis), np.min),
      f"{prefix}/max": (np.max(rewards, axis=axis), np.max),
  }


class AbstractRewardManager(abc.ABC):

  def __init__(self, reward_fns: Union[RewardFn, List[RewardFn]], algo_config: Any):
    self.reward_fns = [reward_fns] if not isinstance(reward_fns, Sequence) else list(reward_fns)
    if not self.reward_fns:
      raise ValueError("reward_fns cannot be empty. You must provide at least one reward function.")
    self.algo_config = algo_config

  @abc.abstractmethod
  def __call__(self, prompts: List[str], completions: List[str], **kwargs) -> Dict[str, Any]:
    ...


def _cfg_dict(cfg) -> Dict[str, Any]:
  if dataclasses.is_dataclass(cfg):
    return {f.name: getattr(cfg, f.name) for f in dataclasses.fields(cfg)}
  return dict(vars(cfg)) if hasattr(cfg, "__dict__") else {}


@function_registry.register_reward_manager("sequence-level")
class SequenceRewardManager(AbstractRewardManager):
  """One scalar reward per sequence: the sum over reward functions."""

  def __init__(self, reward_fns, algo_config, **kwargs):
    super().__init__(reward_fns, algo_config)

  def __call__(self, prompts, completions, **kwargs):
    return self._compute_rewards(prompts, completions, **kwargs)

  def _compute_rewards(self, prompts, completions, **kwargs) -> Dict[str, Any]:
    cfg = _cfg_dict(self.algo_config)
    rewards = np.zeros((len(prompts), len(self.reward_fns)))
    for i, fn in enumerate(self.reward_fns):
      extra = {}
      for name in inspect.signature(fn).parameters:
        if name in ("self", "prompts", "completions", "kwargs"):
          continue
        if name in cfg and name not in kwargs:
          extra[name] = cfg[name]
      r = fn(prompts=prompts, completions=completions, **{**kwargs, **extra})
      name = getattr(fn, "__name__", type(fn).__name__)
      if r is None:
        raise RuntimeError(f"Failed to obtain result from {name}. Result is None.")
      if isinstance(r, list) and len(r) != len(prompts):
        raise RuntimeError(f"Length mismatch after {name}: len(r)={len(r)}, len(prompts)={len(prompts)}. "
                           f"Content of r: {r}")
      rewards[:, i] = np.array(r)
    log_metrics = self._prepare_log_metrics(prompts, completions, rewards)
    info = {"rewards": np.nansum(rewards, axis=1), "log_metrics": log_metrics}
    if os.getenv("TUNIX_DEBUG_REWARDS"):
      log.info("======= example rewards =======")
      for k, v in log_metrics.items():
        s = str(v[0][0])
        log.info("%s:\t%s", k, s if len(s) <= 100 else s[:50] + "..." + s[-50:])
      log.info("=======================")
    return info

  def _prepare_log_metrics(self, prompts, completions, rewards: np.ndarray) -> Dict[str, Any]:
    m: Dict[str, Any] = {"prompts": (prompts, None), "completions": (completions, None)}
    m.update(_calculate_scalar_reward_log_metrics(rewards, prefix="rewards"))
    for i, fn in enumerate(self.reward_fns):
      m[f"rewards/{getattr(fn, '__name__', type(fn).__name__)}"] = (rewards[:, i], np.mean)
    return m


@function_registry.register_reward_manager("agentic-sequence-level")
class AgenticSequenceRewardManager(SequenceRewardManager):
  """Adds environment trajectory rewards (`trajectory_rewards` kwarg) to the optional reward functions."""

  def __init__(self, reward_fns, algo_config, **kwargs):
    if reward_fns is None:
      self.reward_fns = []
      self.algo_config = algo_config
    else:
      super().__init__(reward_fns, algo_config)

  def __call__(self, prompts, completions, **kwargs):
    traj = np.asarray(kwargs.pop("trajectory_rewards"), dtype=np.float64).copy()
    log_metrics = dict(_calculate_scalar_reward_log_metrics(traj, prefix="trajectory_rewards", axis=0))
    final = traj
    if self.reward_fns:
      info = self._compute_rewards(prompts, completions, **kwargs)
      final = final + info["rewards"]
      log_metrics.update(info["log_metrics"])
    return {"rewards": final, "log_metrics": log_metrics}
