"""Rollout through the paged continuous-batching engine (`tunix_b200.rollout.PagedEngine`).

Same contract as the other engines (tunix/rl/rollout/base_rollout.py:35-103): prompts are
tokenised (BOS de-duplicated), truncated on the left to `max_prompt_length`, generated with
temperature sampling with optional top-k / top-p,
and returned with left-padded prompt ids and per-token log-probs of the sampled tokens.
Weights are the rollout model's own parameters, so `update_params` is an in-place copy (or a
no-op when trainer and rollout share parameters) and the KV cache needs no rebuild.
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional, Tuple

import numpy as np
import torch

from ...generate import tokenizer_adapter as tok_adapter
from ...rollout import EngineConfig, PagedEngine
from ...rollout import engine as engine_lib
from .. import common
from . import base_rollout, vanilla_rollout


DEFAULT_MAX_BATCH = 512      # sequences decoded together; lower it when the KV cache must stay small
DEFAULT_PAGE_SIZE = 64       # one TMA box per 64-key tile in the decode kernel


class NativeRollout(base_rollout.BaseRollout):
  def __init__(self, model: torch.nn.Module, tokenizer: Any, rollout_config: base_rollout.RolloutConfig, mesh=None,
               page_size: Optional[int] = None, max_batch: Optional[int] = None):
    page_size = page_size or DEFAULT_PAGE_SIZE
    max_batch = max_batch or DEFAULT_MAX_BATCH
    self._model = model
    self._tokenizer = tokenizer if isinstance(tokenizer, tok_adapter.TokenizerAdapter) else \
        tok_adapter.TokenizerAdapter(tokenizer)
    self._mesh = mesh
    rc = rollout_config
    mc = model.config
    self._fallback = None
    if not engine_lib.supported(mc):
      cache = base_rollout.CacheConfig(cache_size=rc.kv_cache_size, num_layers=mc.num_layers,
                                       num_kv_heads=mc.num_kv_heads, head_dim=mc.head_dim)
      self._fallback = vanilla_rollout.VanillaRollout(model, tokenizer, cache)
      self._engine = None
    else:
      max_seq = max(rc.kv_cache_size, rc.max_prompt_length + rc.max_tokens_to_generate)
      self._engine = PagedEngine(model, EngineConfig(page_size=page_size, max_batch=max_batch, max_seq_len=max_seq,
                                                     use_cuda_graphs=next(model.parameters()).is_cuda))

  def _tokenize(self, s: str) -> List[int]:
    ids = list(self._tokenizer.encode(s))
    bos = self._tokenizer.bos_id()
    if bos:
      ids = list(self._tokenizer.dedup_bos_ids([bos] + ids))
    return ids

  def generate(self, prompts: List[str], rollout_config: base_rollout.RolloutConfig, **kwargs):
    rc = rollout_config
    if self._engine is None:
      fb = self._fallback or vanilla_rollout.VanillaRollout(
          self._model, self._tokenizer, base_rollout.CacheConfig(
              cache_size=rc.kv_cache_size, num_layers=self._model.config.num_layers,
              num_kv_heads=self._model.config.num_kv_heads, head_dim=self._model.config.head_dim))
      self._fallback = fb
      return fb.generate(prompts, rc, **kwargs)
    P = rc.max_prompt_length
    pad = self.pad_id()
    ids = [self._tokenize(p)[-P:] for p in prompts]
    eos = list(rc.eos_tokens) if rc.eos_tokens else [self.eos_id()]
    res = self._engine.generate(ids, rc.max_tokens_to_generate, temperature=rc.temperature or 0.0,
                                greedy=not rc.temperature, seed=rc.seed or 0, eos_ids=eos,
                                return_logprobs=True, top_k=rc.top_k, top_p=rc.top_p)
    tokens, lps = [], []
    for t, l in zip(res.tokens, res.logprobs):
      if len(t) and int(t[-1]) in eos:        # the EOS ends the completion and is not part of it
        t, l = t[:-1], l[:-1]
      tokens.append(np.asarray(t))
      lps.append(np.asarray(l, dtype=np.float32))
    padded = np.full((len(ids), P), pad, dtype=np.int64)
    for i, p in enumerate(ids):
      padded[i, P - len(p):] = p
    text = [self._tokenizer.decode(t.tolist()) for t in tokens]
    return base_rollout.RolloutOutput(text=text, logits=None, tokens=tokens, left_padded_prompt_tokens=padded,
                                      logprobs=lps if rc.return_logprobs else None)

  def get_per_token_logps(self, prompt_tokens, completion_tokens):
    return common.compute_per_token_logps(self._model, prompt_tokens, completion_tokens, self.pad_id(), self.eos_id(),
                                          stop_gradient=True)

  @torch.no_grad()
  def update_params(self, params: Dict[str, torch.Tensor], filter_types: Optional[Tuple[Any, ...]] = None) -> None:
    dst = dict(self._model.named_parameters())
    for n, t in params.items():
      if n not in dst:
        raise KeyError(f"rollout model has no parameter {n}")
      if dst[n].data_ptr() != t.data_ptr():
        dst[n].copy_(t.to(dst[n].device, dst[n].dtype))

  def pad_id(self) -> int:
    return self._tokenizer.pad_id()

  def eos_id(self) -> int:
    return self._tokenizer.eos_id()

  def model(self) -> torch.nn.Module:
    return self._model
