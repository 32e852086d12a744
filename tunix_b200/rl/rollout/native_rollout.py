"""Rollout through the paged continuous-batching engine (`tunix_b200.rollout.PagedEngine`).

Same contract as the other engines (tunix/rl/rollout/base_rollout.py:35-103): prompts are
tokenised (BOS de-duplicated), truncated on the left to `max_prompt_length`, generated with
temperature sampling with optional top-k / top-p,
and returned with left-padded prompt ids and per-token log-probs of the sampled tokens.
Weights are the rollout model's own parameters, so `update_params` is an in-place copy (or a
no-op when trainer and rollout share parameters) and the KV cache needs no rebuild.

Tensor-parallel rollout (`RolloutConfig.tensor_parallel_size` > 1, tunix/common/configs.py:70-256): the
engine runs on a `dist.weight_sync.RolloutReplica` - this rank's tensor-parallel slice of the trainer's
flat parameter store - whose row-parallel exits all-reduce inside the decode GEMM kernel over peer
memory. `update_params` is then one launch of the re-sharding copy kernel. The ranks of a
tensor-parallel group decode the union of their prompts together (same seeds, bitwise-equal reduced
logits, hence the same tokens on every rank) and each keeps the completions of its own prompts.
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
               page_size: Optional[int] = None, max_batch: Optional[int] = None,
               engine_overrides: Optional[dict] = None):
    page_size = page_size or DEFAULT_PAGE_SIZE
    max_batch = max_batch or DEFAULT_MAX_BATCH
    self._model = model
    self._tokenizer = tokenizer if isinstance(tokenizer, tok_adapter.TokenizerAdapter) else \
        tok_adapter.TokenizerAdapter(tokenizer)
    self._mesh = mesh
    rc = rollout_config
    self._replica = None
    self._tp_group, self._tp, self._tp_rank = None, 1, 0
    tp = int(getattr(rc, "tensor_parallel_size", -1) or -1)
    if tp > 1:
      model = self._build_replica(model, tp, mesh)
      self._model = model
    mc = model.config
    self._fallback = None
    if not engine_lib.supported(mc):
      cache = base_rollout.CacheConfig(cache_size=rc.kv_cache_size, num_layers=mc.num_layers,
                                       num_kv_heads=mc.num_kv_heads, head_dim=mc.head_dim)
      self._fallback = vanilla_rollout.VanillaRollout(model, tokenizer, cache)
      self._engine = None
    else:
      max_seq = max(rc.kv_cache_size, rc.max_prompt_length + rc.max_tokens_to_generate)
      extra = {k: v for k, v in (engine_overrides or {}).items() if k in ("max_prefill_tokens", "num_pages", "share_prefix")}
      max_seq = max(max_seq, int((engine_overrides or {}).get("max_seq_len", 0)))
      self._engine = PagedEngine(model, EngineConfig(page_size=page_size, max_batch=max_batch, max_seq_len=max_seq,
                                                     use_cuda_graphs=next(model.parameters()).is_cuda, **extra))

  def _build_replica(self, trainer_model: torch.nn.Module, tp: int, mesh):
    """This rank's tensor-parallel slice of the trainer's weights, as a model of its own."""
    import torch.distributed as dist
    from ...dist import mesh as mesh_lib, weight_sync
    if not (dist.is_available() and dist.is_initialized()):
      raise ValueError("tensor-parallel rollout needs torch.distributed (one process per GPU)")
    if mesh is None or "tp" not in getattr(mesh, "axis_names", ()) or mesh.axis_size("tp") != tp:
      ranks = mesh.ranks() if mesh is not None else list(range(dist.get_world_size()))
      if len(ranks) % tp:
        raise ValueError(f"{len(ranks)} rollout ranks do not divide into tensor-parallel groups of {tp}")
      mesh = mesh_lib.Mesh((len(ranks) // tp, tp), ("dp", "tp"), ranks)
      self._mesh = mesh
    self._replica = weight_sync.RolloutReplica(trainer_model, mesh, "tp")
    self._replica.sync()
    self._tp_group, self._tp, self._tp_rank = mesh.group("tp"), tp, mesh.axis_index("tp")
    return self._replica.model

  def weight_sync_ms(self) -> Optional[float]:
    """Device time of the last trainer -> rollout weight transfer (None: weights are shared in place)."""
    return self._replica.sync_ms() if self._replica is not None else None

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
    all_ids, lo = ids, 0
    if self._tp > 1:
      # the ranks of a tensor-parallel group decode the union of their prompts in one batch
      import torch.distributed as dist
      parts: List[Any] = [None] * self._tp
      dist.all_gather_object(parts, ids, group=self._tp_group)
      lo = sum(len(p) for p in parts[:self._tp_rank])
      all_ids = [p for part in parts for p in part]
    res = self._engine.generate(all_ids, rc.max_tokens_to_generate, temperature=rc.temperature or 0.0,
                                greedy=not rc.temperature, seed=rc.seed or 0, eos_ids=eos,
                                return_logprobs=True, top_k=rc.top_k, top_p=rc.top_p)
    tokens, lps = [], []
    for t, l in zip(res.tokens[lo:lo + len(ids)], res.logprobs[lo:lo + len(ids)]):
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
    if self._tp > 1:
      raise NotImplementedError("score with the trainer's model: the ranks of a tensor-parallel rollout group would "
                                "have to score identical batches")
    return common.compute_per_token_logps(self._model, prompt_tokens, completion_tokens, self.pad_id(), self.eos_id(),
                                          stop_gradient=True)

  @torch.no_grad()
  def update_params(self, params: Dict[str, torch.Tensor], filter_types: Optional[Tuple[Any, ...]] = None) -> None:
    if self._replica is not None:
      self._replica.sync()          # one launch: trainer flat buffer -> this rank's tensor-parallel slice
      return
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
