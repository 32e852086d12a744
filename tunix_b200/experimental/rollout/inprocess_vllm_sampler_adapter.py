"""`Sampler` service over a vLLM engine living in this process (`generate.vllm_sampler.VllmSampler`; the
reference's counterpart is tunix/experimental/rollout/inprocess_vllm_sampler_adapter.py:40-327).

vLLM holds its own copy of the weights in its own layout, so the serving tensors of this adapter are the
*trainer-layout* parameters of a shadow model: a weight sync stages into a copy of those, and publishing streams
them - renamed and split the way the checkpoint exporter does - into the engine's `load_weights`, then resets the
prefix cache (cached prefixes were computed with the old weights). The engine batches continuously by itself, so
requests are simply forwarded with their own sampling parameters."""
from __future__ import annotations

from typing import Any, Dict, List, Optional, Sequence

import numpy as np
import torch

from ...generate import vllm_sampler
from . import sampler as sampler_lib
from . import staged_sampler


class InprocessVllmSamplerAdapter(staged_sampler.StagedSampler):

  def __init__(self, model: torch.nn.Module, tokenizer: Any, *, config: Optional[vllm_sampler.VllmConfig] = None,
               llm: Any = None, handler=None, worker_id: str = "sampler0", rank: int = 0,
               eos_ids: Optional[Sequence[int]] = None):
    """`model` is the trainer-layout model whose parameters define names and shapes of a sync; `llm` injects a
    ready engine (tests, or an engine shared with another sampler)."""
    super().__init__(tokenizer, handler=handler, worker_id=worker_id, rank=rank, eos_ids=eos_ids)
    self._model, self._config, self._llm = model, config or vllm_sampler.VllmConfig(), llm
    self._sampler: Optional[vllm_sampler.VllmSampler] = None

  def initialize(self) -> None:
    if self._sampler is None:
      self._sampler = vllm_sampler.VllmSampler(self._tok, self._config, model=self._model, llm=self._llm)

  def _serving(self) -> Dict[str, torch.Tensor]:
    return staged_sampler.lora_aware_parameters(self._model)

  def _publish(self, staging: Dict[str, torch.Tensor]) -> None:
    self.initialize()
    super()._publish(staging)                         # keep the shadow model equal to what the engine serves
    self._sampler.update_params(dict(self._serving()))

  def _cache_usage_percent(self) -> float:
    probe = getattr(getattr(self._sampler, "llm", None), "kv_cache_usage", None)
    try:
      return 100.0 * float(probe()) if callable(probe) else 0.0
    except Exception:  # noqa: BLE001 - a metric, never a failure
      return 0.0

  def _generate_batch(self, reqs, params: sampler_lib.SamplingParams) -> List[sampler_lib.SamplingResponse]:
    if params.beam_size:
      raise NotImplementedError("beam search is not available through vLLM")
    prompts = [self.prompt_ids(r.prompt) for r in reqs]
    version = self.policy_version
    engine = self._sampler
    sp = engine._sampling_params(params.max_tokens, params.temperature, params.top_p, params.top_k, params.seed,
                                 self._eos, params.return_logprobs)
    outs = engine.generate_ids(prompts, sp)
    answers = []
    for req, prompt, out in zip(reqs, prompts, outs):
      completion = out.outputs[0]
      tokens = np.asarray(list(completion.token_ids), np.int32)
      lps = None
      if params.return_logprobs and getattr(completion, "logprobs", None):
        lps = np.asarray([_chosen_logprob(step, tok) for step, tok in zip(completion.logprobs, tokens)], np.float32)
      reason = getattr(completion, "finish_reason", None)
      hit_eos = reason == "stop" or (bool(len(tokens)) and int(tokens[-1]) in self._eos)
      answers.append(self.response(req, prompt, tokens, lps, hit_eos, version))
    return answers


def _chosen_logprob(step: Any, token: int) -> float:
  """vLLM reports, per step, a dict {token id: Logprob}; plain floats and dict-of-floats are accepted too."""
  if isinstance(step, dict):
    entry = step.get(int(token), next(iter(step.values())))
    return float(getattr(entry, "logprob", entry))
  return float(getattr(step, "logprob", step))
