"""KV-cached batched sampler.

Same contract as tunix/generate/sampler.py:198-1011: prompts are tokenised (BOS de-duplicated),
left-padded to `max_prompt_length` (next power of two when unset), prefilled in one forward pass
and decoded one token per step until every row has emitted an EOS id or the step budget is used
up; greedy, top-p (+ top-k) with temperature, or beam search; optional per-step logits and
log-probabilities (always of the unfiltered, temperature-scaled distribution); forbidden tokens;
`echo` and `pad_output`.

The sampling key of step s is derived from `(seed, s)`, so a run is reproducible and independent
of batch composition. This class keeps the reference's static batch and contiguous cache; the
continuous-batching engine with a paged cache lives in `tunix_b200.rollout`.
"""
from __future__ import annotations

import dataclasses
from typing import Any, Dict, Iterable, List, Optional, Sequence, Union

import numpy as np
import torch

from ..common.configs import CacheConfig
from . import base_sampler, beam_search as beam_lib, tokenizer_adapter as tok_adapter, utils

SamplerOutput = base_sampler.SamplerOutput


def _step_generator(seed: int, step: int, device) -> torch.Generator:
  g = torch.Generator(device=device)
  g.manual_seed((int(seed) * 1_000_003 + int(step) * 7919 + 12345) % (2 ** 63 - 1))
  return g


def sample_top_p(logits: torch.Tensor, gen: torch.Generator, temperature: float, top_p: float, top_k: Optional[int],
                 return_logprobs: bool = False):
  """logits [B, V] -> (token [B], logprob [B] or None). The top-p mask keeps the smallest prefix
  of the (top-k) sorted distribution whose preceding mass is <= top_p."""
  z = logits.float() / temperature
  no_topk = top_k is None or top_k <= 0
  if top_p >= 1.0 and no_topk:
    tok = torch.multinomial(torch.softmax(z, dim=-1), 1, generator=gen).squeeze(-1)
  else:
    k = z.shape[-1] if no_topk else min(int(top_k), z.shape[-1])
    zs, idx = torch.topk(z, k, dim=-1)
    ps = torch.softmax(zs, dim=-1)
    cum = torch.cumsum(ps, dim=-1)
    zs = torch.where(cum - ps > top_p, torch.full_like(zs, float("-inf")), zs)
    pick = torch.multinomial(torch.softmax(zs, dim=-1), 1, generator=gen)
    tok = idx.gather(-1, pick).squeeze(-1)
  lp = None
  if return_logprobs:
    lp = torch.log_softmax(z, dim=-1).gather(-1, tok[:, None]).squeeze(-1)
  return tok, lp


def sample_best(logits: torch.Tensor, return_logprobs: bool = False):
  tok = torch.argmax(logits, dim=-1)
  lp = None
  if return_logprobs:
    lp = torch.log_softmax(logits.float(), dim=-1).gather(-1, tok[:, None]).squeeze(-1)
  return tok, lp


class Sampler(base_sampler.BaseSampler):
  """Sampler for a decoder with the `Transformer` call contract."""

  def __init__(self, transformer: torch.nn.Module, tokenizer: Any, cache_config: CacheConfig,
               image_processor: Any = None):
    self.tokenizer = tokenizer if isinstance(tokenizer, tok_adapter.TokenizerAdapter) else \
        tok_adapter.TokenizerAdapter(tokenizer)
    self.cache_config = cache_config
    self.image_processor = image_processor
    self._transformer = transformer

  # ---- model state ---------------------------------------------------------------------
  @property
  def transformer(self) -> torch.nn.Module:
    return self._transformer

  @property
  def transformer_state(self) -> Dict[str, torch.Tensor]:
    return {n: p for n, p in self._transformer.named_parameters()}

  @transformer_state.setter
  def transformer_state(self, state: Dict[str, torch.Tensor]) -> None:
    """Replaces all parameters, or only the LoRA parameters, after checking names, shapes and dtypes."""
    cur = dict(self._transformer.named_parameters())
    lora = {n for n, p in cur.items() if getattr(p, "is_lora", False)}
    keys = set(state.keys())
    if keys != set(cur.keys()) and not (lora and keys == lora):
      missing, extra = set(cur) - keys, keys - set(cur)
      raise ValueError(f"New state must cover all parameters or exactly the LoRA parameters. Missing: "
                       f"{sorted(missing)[:5]}, unexpected: {sorted(extra)[:5]}")
    with torch.no_grad():
      for n, t in state.items():
        p = cur[n]
        if tuple(t.shape) != tuple(p.shape):
          raise ValueError(f"shape mismatch for {n}: {tuple(t.shape)} vs {tuple(p.shape)}")
        if t.dtype != p.dtype:
          raise ValueError(f"dtype mismatch for {n}: {t.dtype} vs {p.dtype}")
        p.copy_(t)

  @property
  def dtype(self) -> torch.dtype:
    return next(self._transformer.parameters()).dtype

  @property
  def device(self) -> torch.device:
    return next(self._transformer.parameters()).device

  def tokenize(self, input_string: str) -> np.ndarray:
    ids = self.tokenizer.encode(input_string)
    bos = [self.tokenizer.bos_id()] if self.tokenizer.bos_id() else []
    return np.array(self.tokenizer.dedup_bos_ids(bos + list(ids)), dtype=np.int32)

  # ---- sampling ------------------------------------------------------------------------------
  def _sample(self, logits: torch.Tensor, step: int, mode: str, temperature: float, top_p, top_k, seed: int,
              forbidden: Optional[Sequence[int]], want_lp: bool):
    if forbidden:
      logits = logits.clone()
      logits[:, list(forbidden)] = float("-inf")
    if mode == "greedy":
      return sample_best(logits, want_lp)
    return sample_top_p(logits, _step_generator(seed, step, logits.device), temperature, top_p, top_k, want_lp)

  @torch.no_grad()
  def __call__(self, input_strings: Union[str, Sequence[str]], max_generation_steps: int,
               max_prompt_length: Optional[int] = None, echo: bool = False, return_logits: bool = False,
               return_logprobs: bool = False, eos_tokens: Optional[Sequence[int]] = None,
               forbidden_tokens: Optional[Iterable[int]] = None, temperature: float = 0.0,
               top_p: Optional[float] = None, top_k: Optional[int] = None, beam_size: Optional[int] = None,
               seed: Optional[int] = None, pad_output: bool = False, images=None, audios=None,
               max_audio_length=None, max_audio_clips=None) -> SamplerOutput:
    """Samples completions. Mode: beam search if `beam_size`, top-p if `top_p` (or top_k) is
    given with a non-zero temperature, else greedy."""
    del images, audios, max_audio_length, max_audio_clips   # text-only decoder
    model = self._transformer
    dev = self.device
    eos_ids = list(eos_tokens) if eos_tokens else [self.tokenizer.eos_id()]
    strings = [input_strings] if isinstance(input_strings, str) else list(input_strings)
    forbidden = tuple(forbidden_tokens) if forbidden_tokens else None
    toks = [self.tokenize(s) for s in strings]
    longest = max(len(t) for t in toks)
    if max_prompt_length is None or max_prompt_length < longest:
      max_prompt_length = utils.next_power_of_2(longest)
    P = int(max_prompt_length)
    pad = self.tokenizer.pad_id()
    prompts = np.full((len(toks), P), pad, dtype=np.int64)
    for i, t in enumerate(toks):
      t = t[-P:]
      prompts[i, P - len(t):] = t
    total = P + int(max_generation_steps)
    if total > self.cache_config.cache_size:
      raise ValueError(f"Total sampling steps {total} must be less than the cache size "
                       f"{self.cache_config.cache_size}.")
    if beam_size:
      mode = "beam_search"
    elif (top_p is not None or top_k) and temperature and temperature > 0:
      mode = "top_p"
      top_p = 1.0 if top_p is None else top_p
    else:
      mode = "greedy"
    seed = 0 if seed is None else int(seed)
    if mode == "beam_search":
      return beam_lib.run_beam_search(self, prompts, P, max_generation_steps, beam_size, eos_ids, pad, echo,
                                      return_logits, return_logprobs, pad_output)

    B = prompts.shape[0]
    S = self.cache_config.cache_size
    buf = torch.full((B, total), pad, dtype=torch.long, device=dev)
    buf[:, :P] = torch.from_numpy(prompts).to(dev)
    valid = buf != pad
    valid[:, P:] = True
    positions = torch.cumsum(valid.long(), dim=-1)
    positions = positions - (positions >= 1).long()
    cache = model.init_cache(B, S, dtype=self.dtype, device=dev)
    V = getattr(model, "num_embed", None) or model.config.vocab_size
    logits_buf = torch.zeros(B, total, V, dtype=torch.float32, device=dev) if return_logits else None
    lp_buf = torch.zeros(B, total, dtype=torch.float32, device=dev) if return_logprobs else None
    eos_t = torch.tensor(eos_ids, device=dev)

    # prefill: queries = prompt positions, keys = cache slots [0, S)
    pmask = utils.make_prefill_attention_mask(valid[:, :P], S)
    logits, cache = model(buf[:, :P], positions[:, :P], cache, pmask)
    if echo and return_logits:
      logits_buf[:, 1:P] = logits[:, :-1].float()
    step_logits = logits[:, -1].float()
    done = torch.zeros(B, dtype=torch.bool, device=dev)
    for step in range(P, total):
      tok, lp = self._sample(step_logits, step - P, mode, temperature or 1.0, top_p, top_k, seed, forbidden,
                             return_logprobs)
      tok = torch.where(done, torch.full_like(tok, pad), tok)
      buf[:, step] = tok
      if return_logits:
        logits_buf[:, step] = step_logits
      if return_logprobs:
        lp_buf[:, step] = torch.where(done, torch.zeros_like(lp), lp)
      done = done | torch.isin(tok, eos_t)
      if step == total - 1 or bool(done.all()):
        break
      dmask = utils.make_decode_attention_mask(valid, step, S)
      logits, cache = model(buf[:, step:step + 1], positions[:, step:step + 1], cache, dmask)
      step_logits = logits[:, -1].float()

    return self._finalize(buf.cpu().numpy(), logits_buf, lp_buf, prompts, P, max_generation_steps, total, eos_ids,
                          pad, echo, return_logits, return_logprobs, pad_output)

  def _finalize(self, token_buffers: np.ndarray, logits_buf, lp_buf, prompts, P, max_gen, total, eos_ids, pad, echo,
                return_logits, return_logprobs, pad_output) -> SamplerOutput:
    out_tokens, out_logits, out_lps = [], [], []
    lp_np = lp_buf.cpu().numpy() if lp_buf is not None else None
    for i in range(token_buffers.shape[0]):
      tb = token_buffers[i]
      start = utils.np_find_first_non_pad_idx(tb, pad) if echo else P
      end = utils.np_find_first_eos_idx(tb[P:], eos_ids) + P
      out_tokens.append(tb[start:end])
      if return_logits:
        out_logits.append(logits_buf[i, start:end].cpu())
      if return_logprobs:
        out_lps.append(lp_np[i, start:end].tolist())
    text = [self.tokenizer.decode(t.tolist()) for t in out_tokens]
    if pad_output:
      max_len = total if echo else max_gen
      padded = np.full((len(out_tokens), max_len), pad, dtype=token_buffers.dtype)
      for i, t in enumerate(out_tokens):
        padded[i, :len(t)] = t
      if return_logprobs:
        out_lps = [l + [0.0] * (max_len - len(l)) for l in out_lps]
      if return_logits:
        out_logits = [torch.nn.functional.pad(l, (0, 0, 0, max_len - l.shape[0])) for l in out_logits]
        out_logits = torch.stack(out_logits)
      out_tokens = padded
    return SamplerOutput(text=text, logits=out_logits if return_logits else [], tokens=out_tokens,
                         padded_prompt_tokens=prompts, logprobs=out_lps if return_logprobs else None)
