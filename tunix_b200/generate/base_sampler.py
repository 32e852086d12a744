"""Sampler interface and output record (tunix/generate/base_sampler.py:31-88)."""
from __future__ import annotations

import abc
import dataclasses
from typing import Any, List, Optional, Union

import numpy as np


@dataclasses.dataclass
class SamplerOutput:
  text: List[str]                       # decoded completions
  logits: Any                           # per-step logits when requested, else []
  tokens: Any                           # generated ids per sample (list of arrays, or padded array)
  padded_prompt_tokens: np.ndarray      # left-padded prompt ids [B, max_prompt_length]
  logprobs: Optional[List[List[float]]]  # log-probability of every sampled token when requested


class BaseSampler(abc.ABC):

  @property
  @abc.abstractmethod
  def transformer(self):
    ...

  @property
  @abc.abstractmethod
  def transformer_state(self):
    ...

  @abc.abstractmethod
  def __call__(self, input_strings, max_generation_steps, max_prompt_length=None, temperature=0.0, top_p=None,
               top_k=None, beam_size=None, seed=None, multi_sampling: int = 1, return_logits: bool = True,
               echo: bool = False, pad_output: bool = False):
    ...

  @abc.abstractmethod
  def tokenize(self, input_string: str):
    ...
