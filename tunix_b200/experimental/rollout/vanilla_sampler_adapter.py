"""`Sampler` service over the dense-cache sampler (`generate.sampler.Sampler`: static batch, contiguous KV cache;
the reference's counterpart is tunix/experimental/rollout/vanilla_sampler_adapter.py:40-342).

Use it where the paged engine does not apply - models with image or audio inputs, beam search, per-step logits - or
as the simple baseline engine. Requests of one call are generated as one static batch per distinct sampling
setting; prompts are passed as token ids when given as ids, and the sampler's own tokenisation is bypassed for
them by decoding-free id injection (`Sampler.tokenize` is only used for text prompts)."""
from __future__ import annotations

from typing import Any, Dict, List, Optional, Sequence

import numpy as np
import torch

from ...generate import sampler as dense_sampler
from . import sampler as sampler_lib
from . import staged_sampler


class VanillaSamplerAdapter(staged_sampler.StagedSampler):

  def __init__(self, model: torch.nn.Module, tokenizer: Any, *, cache_config: Optional[dense_sampler.CacheConfig] = None,
               max_prompt_length: Optional[int] = None, handler=None, worker_id: str = "sampler0", rank: int = 0,
               eos_ids: Optional[Sequence[int]] = None):
    super().__init__(tokenizer, handler=handler, worker_id=worker_id, rank=rank, eos_ids=eos_ids)
    self._model = model
    self._cache_config = cache_config
    self._max_prompt_length = max_prompt_length
    self._sampler: Optional[dense_sampler.Sampler] = None

  def initialize(self) -> None:
    if self._sampler is not None:
      return
    cfg = self._cache_config
    if cfg is None:
      mc = self._model.config
      cfg = dense_sampler.CacheConfig(cache_size=4096, num_layers=mc.num_layers, num_kv_heads=mc.num_kv_heads,
                                      head_dim=mc.head_dim)
    self._sampler = dense_sampler.Sampler(self._model, self._tok, cfg)

  def _serving(self) -> Dict[str, torch.Tensor]:
    return staged_sampler.lora_aware_parameters(self._model)

  def _publish(self, staging: Dict[str, torch.Tensor]) -> None:
    self.initialize()
    self._sampler.transformer_state = staging        # validates names, shapes and dtypes, then copies in place

  def _generate_batch(self, reqs, params: sampler_lib.SamplingParams) -> List[sampler_lib.SamplingResponse]:
    prompts = [self.prompt_ids(r.prompt) for r in reqs]
    version = self.policy_version
    out = _IdPrompts(self._sampler, prompts)(
        max_generation_steps=params.max_tokens, max_prompt_length=self._max_prompt_length,
        return_logprobs=params.return_logprobs, return_logits=params.return_logits, eos_tokens=self._eos,
        temperature=params.temperature, top_p=params.top_p, top_k=params.top_k, beam_size=params.beam_size,
        seed=params.seed)
    answers = []
    for i, (req, prompt) in enumerate(zip(reqs, prompts)):
      tokens = np.asarray(out.tokens[i], np.int32)
      hit_eos = bool(len(tokens)) and int(tokens[-1]) in self._eos
      lps = np.asarray(out.logprobs[i], np.float32) if params.return_logprobs and out.logprobs is not None else None
      if lps is not None and lps.shape != tokens.shape:
        lps = lps[:len(tokens)]
      answers.append(self.response(req, prompt, tokens, lps, hit_eos or len(tokens) < params.max_tokens, version))
    return answers


class _IdPrompts:
  """Calls a dense sampler with prompts that are already token ids: for the length of the call the sampler's
  `tokenize` hands back the prepared ids in order."""

  def __init__(self, sampler: dense_sampler.Sampler, prompts: Sequence[Sequence[int]]):
    self.sampler, self.prompts = sampler, [np.asarray(p, np.int32) for p in prompts]

  def __call__(self, **kwargs):
    queue = iter(self.prompts)
    original = self.sampler.tokenize
    self.sampler.tokenize = lambda _text: next(queue)        # type: ignore[method-assign]
    try:
      return self.sampler([""] * len(self.prompts), **kwargs)
    finally:
      self.sampler.tokenize = original                        # type: ignore[method-assign]
