"""Rollout through vLLM (tunix/rl/rollout/vllm_rollout.py:27-146). Optional: needs the `vllm`
package; the adapter lives in `tunix_b200.generate.vllm_sampler`."""
from __future__ import annotations

from typing import Any, Dict, List, Optional, Tuple

import torch

from .. import common
from . import base_rollout


class VllmRollout(base_rollout.BaseRollout):
  holds_own_weights = True       # the engine keeps a copy in its own layout: every optimizer step must be pushed to it

  def __init__(self, model: Any, tokenizer: Any, rollout_config: base_rollout.RolloutConfig, mesh=None,
               cache_config_or_size: Any = None):
    from ...generate import vllm_sampler
    self._model = model
    self._sampler = vllm_sampler.VllmSampler(tokenizer=tokenizer, config=vllm_sampler.VllmConfig.from_rollout_config(
        rollout_config, mesh=mesh), model=model)

  def generate(self, prompts: List[str], rollout_config: base_rollout.RolloutConfig, **kwargs):
    rc = rollout_config
    out = self._sampler(input_strings=prompts, max_generation_steps=rc.max_tokens_to_generate,
                        max_prompt_length=rc.max_prompt_length, temperature=rc.temperature, top_p=rc.top_p,
                        top_k=rc.top_k, seed=rc.seed, echo=False, pad_output=False, eos_tokens=rc.eos_tokens,
                        return_logprobs=rc.return_logprobs)
    return base_rollout.RolloutOutput(text=out.text, logits=None, tokens=out.tokens,
                                      left_padded_prompt_tokens=out.padded_prompt_tokens, logprobs=out.logprobs)

  def get_per_token_logps(self, prompt_tokens, completion_tokens):
    return common.compute_per_token_logps(self._model, prompt_tokens, completion_tokens, self.pad_id(), self.eos_id(),
                                          stop_gradient=True)

  def update_params(self, params: Dict[str, torch.Tensor], filter_types: Optional[Tuple[Any, ...]] = None) -> None:
    self._sampler.update_params(params, filter_types)

  def pad_id(self) -> int:
    return self._sampler.tokenizer.pad_id()

  def eos_id(self) -> int:
    return self._sampler.tokenizer.eos_id()

  def model(self) -> Any:
    return self._model
