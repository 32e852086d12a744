"""A rollout engine that fabricates completions: random token ids with a configurable length
distribution and latency. For tests and for exercising the learner pipeline without a model
(tunix/rl/rollout/mock_rollout.py:40-345)."""
from __future__ import annotations

import dataclasses
import time
from typing import Any, Callable, List, Optional, Sequence, Tuple

import numpy as np
import torch

from . import base_rollout


@dataclasses.dataclass
class MockRolloutConfig:
  vocab_size: int = 1000
  min_length: int = 1
  max_length: Optional[int] = None       # defaults to rollout_config.max_tokens_to_generate
  length_distribution: str = "uniform"   # "uniform" | "fixed" | "geometric"
  latency_s: float = 0.0
  latency_per_token_s: float = 0.0
  seed: int = 0
  eos_probability: float = 0.0


class MockRollout(base_rollout.BaseRollout):

  def __init__(self, tokenizer: Any = None, config: Optional[MockRolloutConfig] = None, model: Any = None, **kwargs):
    self._tok = tokenizer
    self.config = config or MockRolloutConfig()
    self._model = model
    self._rng = np.random.default_rng(self.config.seed)
    self.num_calls = 0
    self.updated_params = 0

  def _length(self, max_len: int) -> int:
    c = self.config
    hi = min(c.max_length or max_len, max_len)
    lo = min(c.min_length, hi)
    if c.length_distribution == "fixed":
      return hi
    if c.length_distribution == "geometric":
      return int(min(hi, lo + self._rng.geometric(0.1) - 1))
    return int(self._rng.integers(lo, hi + 1))

  def _encode(self, s: str) -> List[int]:
    if self._tok is not None:
      return list(self._tok.encode(s))
    return [1 + (ord(ch) % (self.config.vocab_size - 1)) for ch in s]

  def _decode(self, ids) -> str:
    if self._tok is not None:
      return self._tok.decode(list(ids))
    return " ".join(str(int(i)) for i in ids)

  def generate(self, prompts: List[str], rollout_config: base_rollout.RolloutConfig, **kwargs):
    self.num_calls += 1
    P = rollout_config.max_prompt_length
    pad = self.pad_id()
    left = np.full((len(prompts), P), pad, dtype=np.int64)
    toks, texts, lps = [], [], []
    n_total = 0
    for i, p in enumerate(prompts):
      ids = self._encode(p)[-P:]
      left[i, P - len(ids):] = ids
      n = self._length(rollout_config.max_tokens_to_generate)
      t = self._rng.integers(3, self.config.vocab_size, size=n).astype(np.int64)
      toks.append(t)
      texts.append(self._decode(t))
      lps.append(np.log(self._rng.uniform(0.05, 1.0, size=n)).astype(np.float32))
      n_total += n
    delay = self.config.latency_s + self.config.latency_per_token_s * n_total
    if delay > 0:
      time.sleep(delay)
    return base_rollout.RolloutOutput(text=texts, logits=None, tokens=toks, left_padded_prompt_tokens=left,
                                      logprobs=lps if rollout_config.return_logprobs else None)

  def get_per_token_logps(self, prompt_tokens, completion_tokens):
    return torch.zeros(completion_tokens.shape, dtype=torch.float32)

  def update_params(self, params, filter_types=None) -> None:
    self.updated_params += 1

  def pad_id(self) -> int:
    return self._tok.pad_id() if self._tok is not None else 0

  def eos_id(self) -> int:
    return self._tok.eos_id() if self._tok is not None else 2

  def model(self):
    return self._model
