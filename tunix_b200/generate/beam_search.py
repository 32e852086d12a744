"""Batched beam search on top of the sampler's KV-cached forward
(tunix/generate/beam_search.py:27-305): the prompt is prefilled once per row, caches and token
buffers are repeated `beam` times, every step keeps the top-`beam` of `beam * V` continuations
per row and gathers the caches by parent beam; finished beams keep their score and emit padding;
the best beam per row is returned."""
from __future__ import annotations

from typing import List, Sequence

import numpy as np
import torch

from . import utils


def _gather_cache(cache, idx: torch.Tensor):
  return {name: {"k": c["k"].index_select(0, idx), "v": c["v"].index_select(0, idx),
                 "end_index": c["end_index"].index_select(0, idx)} for name, c in cache.items()}


@torch.no_grad()
def run_beam_search(sampler, prompts: np.ndarray, P: int, max_generation_steps: int, beam_size: int,
                    eos_ids: Sequence[int], pad: int, echo: bool, return_logits: bool, return_logprobs: bool,
                    pad_output: bool):
  model, dev = sampler.transformer, sampler.device
  B = prompts.shape[0]
  W = int(beam_size)
  S = sampler.cache_config.cache_size
  total = P + int(max_generation_steps)
  buf = torch.full((B, total), pad, dtype=torch.long, device=dev)
  buf[:, :P] = torch.from_numpy(prompts).to(dev)
  valid = buf != pad
  valid[:, P:] = True
  positions = torch.cumsum(valid.long(), -1)
  positions = positions - (positions >= 1).long()
  cache = model.init_cache(B, S, dtype=sampler.dtype, device=dev)
  logits, cache = model(buf[:, :P], positions[:, :P], cache, utils.make_prefill_attention_mask(valid[:, :P], S))
  logp = torch.log_softmax(logits[:, -1].float(), dim=-1)                # [B, V]
  V = logp.shape[-1]
  # expand to beams
  rep = torch.arange(B, device=dev).repeat_interleave(W)
  buf, valid, positions = buf[rep], valid[rep], positions[rep]
  cache = _gather_cache(cache, rep)
  scores = torch.zeros(B, W, device=dev)
  scores[:, 1:] = float("-inf")                                           # all beams start identical
  done = torch.zeros(B * W, dtype=torch.bool, device=dev)
  lp_buf = torch.zeros(B * W, total, device=dev)
  eos_t = torch.tensor(list(eos_ids), device=dev)
  step_logp = logp[rep]                                                   # [B*W, V]
  for step in range(P, total):
    cand = step_logp.view(B, W, V)
    # finished beams may only continue with padding at no cost
    fin = done.view(B, W)
    cand = torch.where(fin[:, :, None], torch.full_like(cand, float("-inf")), cand)
    cand[:, :, pad] = torch.where(fin, torch.zeros_like(scores), cand[:, :, pad])
    tot = (scores[:, :, None] + cand).view(B, W * V)
    top, flat = torch.topk(tot, W, dim=-1)
    parent = flat // V
    tok = flat % V
    gidx = (torch.arange(B, device=dev)[:, None] * W + parent).view(-1)
    buf, valid, positions, done, lp_buf = buf[gidx], valid[gidx], positions[gidx], done[gidx], lp_buf[gidx]
    cache = _gather_cache(cache, gidx)
    tok = tok.view(-1)
    tok = torch.where(done, torch.full_like(tok, pad), tok)
    buf[:, step] = tok
    lp_buf[:, step] = torch.where(done, torch.zeros_like(top.view(-1)), top.view(-1) - scores.view(-1)[gidx])
    scores = top
    done = done | torch.isin(tok, eos_t)
    if step == total - 1 or bool(done.all()):
      break
    logits, cache = model(buf[:, step:step + 1], positions[:, step:step + 1], cache,
                          utils.make_decode_attention_mask(valid, step, S))
    step_logp = torch.log_softmax(logits[:, -1].float(), dim=-1)
  best = scores.argmax(dim=-1)
  sel = torch.arange(B, device=dev) * W + best
  return sampler._finalize(buf[sel].cpu().numpy(), None, lp_buf[sel] if return_logprobs else None, prompts, P,
                           max_generation_steps, total, eos_ids, pad, echo, False, return_logprobs, pad_output)
