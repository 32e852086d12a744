"""Rollout engine interface (tunix/rl/rollout/base_rollout.py:35-103)."""
from __future__ import annotations

import abc
import dataclasses
from typing import Any, List, Optional, Tuple

import numpy as np

from ...common.configs import CacheConfig, RolloutConfig  # noqa: F401  (re-exported)


@dataclasses.dataclass
class RolloutOutput:
  text: List[str]
  logits: Any
  tokens: List[np.ndarray]
  left_padded_prompt_tokens: np.ndarray
  logprobs: Optional[List[np.ndarray]]


class BaseRollout(abc.ABC):
  # True for engines that keep their own copy of the weights (another process, another layout): the learner then
  # pushes the actor's parameters after every optimizer step even if `model()` returns the actor itself.
  holds_own_weights = False

  @abc.abstractmethod
  def __init__(self, **kwargs):
    ...

  @abc.abstractmethod
  def generate(self, prompts: List[str], rollout_config: RolloutConfig, **kwargs) -> RolloutOutput:
    ...

  @abc.abstractmethod
  def get_per_token_logps(self, prompt_tokens, completion_tokens):
    ...

  @abc.abstractmethod
  def update_params(self, params: Any, filter_types: Optional[Tuple[Any, ...]] = None) -> None:
    ...

  @abc.abstractmethod
  def pad_id(self) -> int:
    ...

  @abc.abstractmethod
  def eos_id(self) -> int:
    ...

  @abc.abstractmethod
  def model(self) -> Any:
    ...
