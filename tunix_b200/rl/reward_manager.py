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


def _summary(values: np.ndarray, prefix: str, axis: int) -> Dict[str, Any]:
  """(values, reducer) pairs for the four summary statistics logged per step."""
  return {f"{prefix}/sum": (np.nansum(values, axis=axis), np.mean), f"{prefix}/mean": (np.nanmean(values, axis=axis), np.mean),
          f"{prefix}/min": (np.min(values, axis=axis), np.min), f"{prefix}/max": (np.max(values, axis=axis), np.max)}


def _config_fields(cfg) -> Dict[str, Any]:
  if dataclasses.is_dataclass(cfg):
    return {f.name: getattr(cfg, f.name) for f in dataclasses.fields(cfg)}
  return dict(vars(cfg)) if hasattr(cfg, "__dict__") else {}


class _BoundReward:
  """A reward function with its calling convention worked out once: which algorithm-config fields it
  asks for by name (they are passed unless the batch already carries a column of that name)."""

  _RESERVED = ("self", "prompts", "completions", "kwargs")

  def __init__(self, fn: RewardFn):
    self.fn = fn
    self.name = getattr(fn, "__name__", type(fn).__name__)
    try:
      params = inspect.signature(fn).parameters
    except (TypeError, ValueError):
      params = {}
    self.wanted = tuple(p for p in params if p not in self._RESERVED)

  def __call__(self, prompts, completions, batch_columns: Dict[str, Any], config: Dict[str, Any]) -> np.ndarray:
    from_config = {k: config[k] for k in self.wanted if k in config and k not in batch_columns}
    scores = self.fn(prompts=prompts, completions=completions, **batch_columns, **from_config)
    if scores is None:
      raise RuntimeError(f"Failed to obtain result from {self.name}. Result is None.")
    if isinstance(scores, list) and len(scores) != len(prompts):
      raise RuntimeError(f"Length mismatch after {self.name}: len(r)={len(scores)}, len(prompts)={len(prompts)}. "
                         f"Content of r: {scores}")
    return np.asarray(scores)


class AbstractRewardManager(abc.ABC):

  def __init__(self, reward_fns: Union[RewardFn, List[RewardFn]], algo_config: Any):
    self.reward_fns = [reward_fns] if not isinstance(reward_fns, Sequence) else list(reward_fns)
    if not self.reward_fns:
      raise ValueError("reward_fns cannot be empty. You must provide at least one reward function.")
    self.algo_config = algo_config

  @abc.abstractmethod
  def __call__(self, prompts: List[str], completions: List[str], **kwargs) -> Dict[str, Any]:
    """-> {"rewards": [B] array, "log_metrics": {name: (values, reducer)}}"""


@function_registry.register_reward_manager("sequence-level")
class SequenceRewardManager(AbstractRewardManager):
  """One scalar reward per sequence: the sum over reward functions."""

  def __init__(self, reward_fns, algo_config, **kwargs):
    super().__init__(reward_fns, algo_config)

  def __call__(self, prompts, completions, **kwargs):
    return self._compute_rewards(prompts, completions, **kwargs)

  def _bound(self) -> List[_BoundReward]:
    cached = getattr(self, "_bound_cache", None)
    if cached is None or [b.fn for b in cached] != list(self.reward_fns):
      cached = self._bound_cache = [_BoundReward(fn) for fn in self.reward_fns]
    return cached

  def _compute_rewards(self, prompts, completions, **kwargs) -> Dict[str, Any]:
    config = _config_fields(self.algo_config)
    bound = self._bound()
    table = np.zeros((len(prompts), len(bound)))           # [sequence, reward function]
    for column, reward in enumerate(bound):
      table[:, column] = reward(prompts, completions, kwargs, config)
    log_metrics: Dict[str, Any] = {"prompts": (prompts, None), "completions": (completions, None)}
    log_metrics.update(_summary(table, "rewards", axis=1))
    for column, reward in enumerate(bound):
      log_metrics[f"rewards/{reward.name}"] = (table[:, column], np.mean)
    if os.getenv("TUNIX_DEBUG_REWARDS"):
      for k, v in log_metrics.items():
        text = str(v[0][0])
        log.info("reward sample %s: %s", k, text if len(text) <= 100 else text[:50] + "..." + text[-50:])
    return {"rewards": np.nansum(table, axis=1), "log_metrics": log_metrics}


@function_registry.register_reward_manager("agentic-sequence-level")
class AgenticSequenceRewardManager(SequenceRewardManager):
  """Environment trajectory rewards (`trajectory_rewards` keyword) plus the optional reward functions."""

  def __init__(self, reward_fns, algo_config, **kwargs):
    if reward_fns is None:
      self.reward_fns, self.algo_config = [], algo_config
    else:
      super().__init__(reward_fns, algo_config)

  def __call__(self, prompts, completions, **kwargs):
    from_env = np.array(kwargs.pop("trajectory_rewards"), dtype=np.float64)
    out = {"rewards": from_env, "log_metrics": _summary(from_env, "trajectory_rewards", axis=0)}
    if self.reward_fns:
      scored = self._compute_rewards(prompts, completions, **kwargs)
      out["rewards"] = from_env + scored["rewards"]
      out["log_metrics"].update(scored["log_metrics"])
    return out
