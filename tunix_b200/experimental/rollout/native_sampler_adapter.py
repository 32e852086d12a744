"""`Sampler` service over the paged engine (continuous batching, paged KV cache, CUDA-graph decode). Lifecycle,
admission and the weight-sync phases come from `staged_sampler.StagedSampler`; the engine reads the model's own
parameter tensors, so publishing staged weights is an in-place copy."""
from __future__ import annotations

from typing import Any, Dict, List, Optional, Sequence

import torch

from ...rollout import EngineConfig, PagedEngine
from . import sampler as sampler_lib
from . import staged_sampler


class NativeSamplerAdapter(staged_sampler.StagedSampler):

  def __init__(self, model: torch.nn.Module, tokenizer: Any, *, engine_config: Optional[EngineConfig] = None,
               handler=None, worker_id: str = "sampler0", rank: int = 0, eos_ids: Optional[Sequence[int]] = None):
    super().__init__(tokenizer, handler=handler, worker_id=worker_id, rank=rank, eos_ids=eos_ids)
    self._model = model
    self._cfg = engine_config or EngineConfig()
    self._engine: Optional[PagedEngine] = None

  def initialize(self) -> None:
    if self._engine is None:
      self._engine = PagedEngine(self._model, self._cfg)

  def _serving(self) -> Dict[str, torch.Tensor]:
    return staged_sampler.lora_aware_parameters(self._model)

  def _cache_usage_percent(self) -> float:
    if self._engine is None:
      return 0.0
    pages = self._engine.cache.allocator
    return 100.0 * (1.0 - pages.free_pages / max(pages.num_pages, 1))

  def _generate_batch(self, reqs, params: sampler_lib.SamplingParams) -> List[sampler_lib.SamplingResponse]:
    prompts = [self.prompt_ids(r.prompt) for r in reqs]
    version = self.policy_version
    extra = {}
    if params.top_k:
      extra["top_k"] = params.top_k
    if params.top_p:
      extra["top_p"] = params.top_p
    res = self._engine.generate(prompts, params.max_tokens, temperature=params.temperature,
                                greedy=params.temperature == 0.0, seed=params.seed or 0, eos_ids=self._eos, **extra)
    return [self.response(r, p, t, lp if params.return_logprobs else None, why == "eos", version)
            for r, p, t, lp, why in zip(reqs, prompts, res.tokens, res.logprobs, res.finish_reasons)]
