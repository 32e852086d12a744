"""Base configuration of RL algorithms with validation (tunix/rl/algorithm_config.py:18-75)."""
from __future__ import annotations

import dataclasses
import logging
from typing import Optional

log = logging.getLogger(__name__)


@dataclasses.dataclass(kw_only=True, slots=True)
class AlgorithmConfig:
  """Fields are keyword-only and the class has slots: a misspelt field is an AttributeError, not a silently ignored
  setting. Values are checked when the object is built; later assignments are not re-checked."""
  algo_variant: str = "grpo"
  advantage_estimator: str = "grpo"
  policy_loss_fn: str = "grpo"
  reward_manager: str = "sequence-level"
  kl_clamp_value: Optional[float] = None

  _valid_algo_variants = ("grpo", "gspo-token", "ppo", "dapo", "drgrpo")
  _valid_advantage_estimators = ("grpo", "gae", "rloo", "drgrpo")
  _valid_policy_loss_fns = ("grpo", "ppo")

  def __post_init__(self):
    if self.algo_variant not in self._valid_algo_variants:
      raise ValueError(f"algo_variant must be one of {list(self._valid_algo_variants)}. Received: "
                       f"{self.algo_variant!r}")
    if self.advantage_estimator not in self._valid_advantage_estimators:
      raise ValueError(f"advantage_estimator must be one of {list(self._valid_advantage_estimators)}. Received: "
                       f"{self.advantage_estimator}")
    if self.policy_loss_fn not in self._valid_policy_loss_fns:
      raise ValueError(f"policy_loss_fn must be one of {list(self._valid_policy_loss_fns)}. Received: "
                       f"{self.policy_loss_fn}")
    self.print_config()

  def print_config(self):
    log.info("Initializing %s:", self.__class__.__name__)
    for f in dataclasses.fields(self):
      log.info("  %s: %s", f.name, getattr(self, f.name))
