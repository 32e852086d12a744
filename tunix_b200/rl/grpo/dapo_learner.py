"""DAPO (https://arxiv.org/pdf/2503.14476): GRPO without a KL term (`beta=None`), asymmetric
clipping (`epsilon_high=0.28`), token-mean aggregation, and overlong-response reward shaping
(tunix/rl/grpo/dapo_learner.py:28-158)."""
from __future__ import annotations

import dataclasses
from typing import Any, Dict, List, Optional, Sequence

from . import grpo_learner as grpo_lib


@dataclasses.dataclass(kw_only=True)
class DAPOConfig(grpo_lib.GRPOConfig):
  algo_variant: str = "dapo"
  advantage_estimator: str = "grpo"
  policy_loss_fn: str = "grpo"
  loss_agg_mode: str = "token-mean"
  reward_manager: str = "sequence-level"
  num_generations: int = 2
  num_iterations: int = 1
  beta: Optional[float] = None
  epsilon: float = 0.2
  epsilon_high: float = 0.28
  dynamic_sampling: bool = True
  overlong_buffer: Optional[Dict[str, Any]] = dataclasses.field(default_factory=lambda: {
      "enable": True, "overlong_buffer_length": 4096, "overlong_buffer_penalty": 1.0, "max_response_length": 20480})

  def __post_init__(self):
    if self.beta is not None:
      raise ValueError("DAPO does not support KL penalty, so beta must be None.")
    if self.epsilon_high < self.epsilon:
      raise ValueError("epsilon_high must be greater than or equal to epsilon.")
    _check_overlong_buffer(self.overlong_buffer)
    super().__post_init__()


_OVERLONG_KEYS = ("overlong_buffer_length", "overlong_buffer_penalty", "max_response_length")


def _check_overlong_buffer(buf: Optional[Dict[str, Any]]) -> None:
  """An enabled buffer must give a positive window, a non-negative penalty and a positive response budget."""
  if not buf or not buf.get("enable"):
    return
  missing = [k for k in _OVERLONG_KEYS if buf.get(k) is None]
  if missing:
    raise ValueError(f"overlong_buffer is enabled but missing: {missing}")
  for key, ok, rule in (("overlong_buffer_penalty", buf["overlong_buffer_penalty"] >= 0, "non-negative"),
                        ("overlong_buffer_length", buf["overlong_buffer_length"] > 0, "positive"),
                        ("max_response_length", buf["max_response_length"] > 0, "positive")):
    if not ok:
      raise ValueError(f"{key} must be {rule}.")


def reward_shaping(prompts: List[str], completions: List[str], mode: Any = None,
                   overlong_buffer: Optional[Dict[str, Any]] = None, **kwargs) -> List[float]:
  """Length penalty of DAPO: a response may use `max_response_length - window` units for free; every unit
  inside the last `window` costs `penalty / window`, so the penalty reaches `-penalty` at the budget (and keeps
  growing beyond it); shorter responses get 0."""
  del prompts, mode, kwargs
  if overlong_buffer is None:
    raise ValueError("reward_shaping is called but with empty overlong_buffer.")
  window, penalty = overlong_buffer["overlong_buffer_length"], overlong_buffer["overlong_buffer_penalty"]
  free = overlong_buffer["max_response_length"] - window
  return [min(0, (free - len(text)) * penalty / window) for text in completions]


class DAPOLearner(grpo_lib.GRPOLearner):

  def __init__(self, rl_engine=None, algo_config: DAPOConfig = None, reward_fns=None,
               metric_fns: Optional[Sequence[Any]] = None, data_shuffle_seed: Optional[int] = None, rl_cluster=None):
    fns = [reward_fns] if not isinstance(reward_fns, Sequence) else list(reward_fns)
    if algo_config.overlong_buffer and algo_config.overlong_buffer["enable"]:
      fns.append(reward_shaping)
    super().__init__(rl_engine=rl_engine, algo_config=algo_config, reward_fns=fns, metric_fns=metric_fns,
                     data_shuffle_seed=data_shuffle_seed, rl_cluster=rl_cluster)


DapoConfig = DAPOConfig
DapoLearner = DAPOLearner
