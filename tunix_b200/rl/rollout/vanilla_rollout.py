"""Rollout through this package's own `Sampler` (tunix/rl/rollout/vanilla_rollout.py:31-130)."""
from __future__ import annotations

import dataclasses
from typing import Any, Dict, List, Optional, Tuple

import torch

from ...generate import sampler as sampler_lib
from .. import common
from . import base_rollout


class VanillaRollout(base_rollout.BaseRollout):

  def __init__(self, model: torch.nn.Module, tokenizer: Any, cache_config_or_size: base_rollout.CacheConfig):
    self._sampler = sampler_lib.Sampler(model, tokenizer, cache_config_or_size)

  def generate(self, prompts: List[str], rollout_config: base_rollout.RolloutConfig, **kwargs):
    out = self._sampler(input_strings=prompts, max_generation_steps=rollout_config.max_tokens_to_generate,
                        max_prompt_length=rollout_config.max_prompt_length, echo=False,
                        temperature=rollout_config.temperature, top_p=rollout_config.top_p,
                        top_k=rollout_config.top_k, seed=rollout_config.seed, pad_output=False,
                        eos_tokens=rollout_config.eos_tokens, return_logprobs=rollout_config.return_logprobs)
    return base_rollout.RolloutOutput(text=out.text, logits=out.logits, tokens=out.tokens,
                                      left_padded_prompt_tokens=out.padded_prompt_tokens, logprobs=out.logprobs)

  def get_per_token_logps(self, prompt_tokens, completion_tokens):
    return common.compute_per_token_logps(self.model(), prompt_tokens, completion_tokens, self.pad_id(),
                                          self.eos_id(), stop_gradient=True)

  @torch.no_grad()
  def update_params(self, params: Dict[str, torch.Tensor], filter_types: Optional[Tuple[Any, ...]] = None) -> None:
    """Copies trainer parameters (all, or the LoRA subset) into the rollout model, casting to its dtype."""
    dst = dict(self.model().named_parameters())
    for n, t in params.items():
      if n not in dst:
        raise KeyError(f"rollout model has no parameter {n}")
      if dst[n].data_ptr() != t.data_ptr():
        dst[n].copy_(t.to(dst[n].device, dst[n].dtype))

  def pad_id(self) -> int:
    return self._sampler.tokenizer.pad_id()

  def eos_id(self) -> int:
    return self._sampler.tokenizer.eos_id()

  def model(self) -> torch.nn.Module:
    return self._sampler.transformer
