"""Continuous-batching generation engine over a paged KV cache.

Requests wait in a queue; between decode steps the scheduler admits as many as fit (pages for
prompt + generation budget are reserved on admission, so a running sequence can never run out
of cache), prefills them - identical prompts once, their samples sharing the prompt's full
pages - and then every running sequence advances one token per step in one batched forward.
Finished sequences free their pages at once and the next waiting requests take their place.

The decode step (model forward + sampling) has fixed shapes per batch-size bucket and is
captured in a CUDA graph per bucket; its inputs live in static device buffers that the
scheduler rewrites before each replay. Sampling uses a counter-based generator keyed by
(seed, step, row), so a run is reproducible.
"""
from __future__ import annotations

import dataclasses
from collections import deque
from typing import Any, Deque, Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..ops import paged
from .paged_cache import OutOfPages, PagedKVCache


@dataclasses.dataclass
class EngineConfig:
  page_size: int = 16
  num_pages: Optional[int] = None          # default: sized from max_batch * max_seq_len
  max_batch: int = 256
  max_seq_len: int = 2048                  # prompt + generation, per sequence
  max_prefill_tokens: int = 16384          # tokens per prefill forward
  use_cuda_graphs: bool = True
  share_prefix: bool = True


@dataclasses.dataclass
class GenerationResult:
  tokens: List[np.ndarray]                 # generated ids per request (EOS included when hit)
  logprobs: Optional[List[np.ndarray]]
  finish_reasons: List[str]                # "eos" | "length"
  steps: int = 0                           # decode forwards that were run
  prefill_ms: float = 0.0                  # device time spent in prompt forwards (CUDA events; 0 on CPU)


@dataclasses.dataclass
class _Seq:
  rid: int
  prompt: Tuple[int, ...]
  max_new: int
  pages: List[int] = dataclasses.field(default_factory=list)
  length: int = 0                          # tokens in the cache
  last_token: int = 0
  out: List[int] = dataclasses.field(default_factory=list)
  lps: List[float] = dataclasses.field(default_factory=list)
  reason: str = ""


def supported(cfg) -> bool:
  """Families whose attention the paged decode kernel covers (no sliding window, no soft-cap)."""
  return not getattr(cfg, "sliding_window_size", None) and not getattr(cfg, "attn_logits_soft_cap", None)


class PagedEngine:
  _max_forbidden = 64       # capacity of the static buffer of never-sampled token ids
  _max_graphs = 16          # captured decode graphs kept (least recently used is dropped)

  def __init__(self, model: torch.nn.Module, config: Optional[EngineConfig] = None):
    self.model = model
    self.cfg = config or EngineConfig()
    mc = model.config
    if not supported(mc):
      raise ValueError("model family needs sliding-window or soft-capped attention, which the paged engine lacks")
    p = next(model.parameters())
    self.device, self.dtype = p.device, p.dtype
    c = self.cfg
    self.max_blocks = (c.max_seq_len + c.page_size - 1) // c.page_size
    num_pages = c.num_pages or (c.max_batch * self.max_blocks + 1)
    self.cache = PagedKVCache(mc.num_layers, num_pages, c.page_size, mc.num_kv_heads, mc.head_dim, self.dtype,
                              self.device)
    self._graphs: Dict[int, Any] = {}
    self._static: Dict[int, Dict[str, torch.Tensor]] = {}
    self._step_counter = torch.zeros((), dtype=torch.int64, device=self.device)
    self._forbidden = torch.zeros(self._max_forbidden, dtype=torch.int32, device=self.device)
    self._num_splits = paged.choose_splits(max(c.max_batch // 4, 1), mc.num_kv_heads, c.max_seq_len)

  # ---- page bookkeeping ----------------------------------------------------------------------
  def _pages_needed(self, seq: _Seq) -> int:
    return self.cache.pages_for(len(seq.prompt) + seq.max_new)

  def _slots(self, seq: _Seq, start: int, n: int) -> List[int]:
    ps = self.cfg.page_size
    return [seq.pages[t // ps] * ps + t % ps for t in range(start, start + n)]

  # ---- prefill -------------------------------------------------------------------------------
  @torch.no_grad()
  def _prefill(self, group: List[_Seq]) -> torch.Tensor:
    """Rows of equal prompt length in one forward; returns last-position logits [B, V]."""
    B, L = len(group), len(group[0].prompt)
    dev = self.device
    tokens = torch.tensor([s.prompt for s in group], dtype=torch.long, device=dev)
    positions = torch.arange(L, device=dev)[None].expand(B, L)
    slots = torch.tensor([x for s in group for x in self._slots(s, 0, L)], dtype=torch.int64, device=dev)
    bt = torch.zeros(B, self.max_blocks, dtype=torch.int32, device=dev)
    lens = torch.full((B,), L, dtype=torch.int32, device=dev)
    caches = self.cache.layer_caches(slots, bt, lens, "prefill")
    hidden, _ = self.model(tokens, positions, caches, None, skip_lm_head=True)
    for s in group:
      s.length = L
    return self.model.compute_final_logits(hidden[:, -1], as_float=False)

  # ---- decode --------------------------------------------------------------------------------
  def _bucket(self, n: int) -> int:
    b = 1
    while b < n:
      b *= 2
    return min(b, max(self.cfg.max_batch, n))

  def _static_buffers(self, bucket: int) -> Dict[str, torch.Tensor]:
    st = self._static.get(bucket)
    if st is None:
      dev = self.device
      st = {"tokens": torch.zeros(bucket, 1, dtype=torch.long, device=dev),
            "positions": torch.zeros(bucket, 1, dtype=torch.long, device=dev),
            "slots": torch.full((bucket,), -1, dtype=torch.int64, device=dev),
            "block_tables": torch.zeros(bucket, self.max_blocks, dtype=torch.int32, device=dev),
            "seq_lens": torch.zeros(bucket, dtype=torch.int32, device=dev)}
      self._static[bucket] = st
    return st

  def _decode_body(self, st: Dict[str, torch.Tensor], sampling: Dict[str, Any]):
    caches = self.cache.layer_caches(st["slots"], st["block_tables"], st["seq_lens"], "decode", self._num_splits,
                                     self.cfg.max_seq_len)
    hidden, _ = self.model(st["tokens"], st["positions"], caches, None, skip_lm_head=True)
    logits = self.model.compute_final_logits(hidden[:, -1], as_float=False)
    return self._sample(logits, sampling)

  def _sample(self, logits: torch.Tensor, sampling: Dict[str, Any]):
    """Greedy / temperature / top-k / top-p sampling in one kernel launch (`ops.paged.sample`). The returned
    log-prob is that of the token under the full tempered distribution, as the trainer recomputes it."""
    return paged.sample(logits, temperature=sampling["temperature"], greedy=sampling["greedy"],
                        seed=sampling["seed"], step=0, step_tensor=self._step_counter,
                        forbidden=self._forbidden, n_forbidden=sampling["n_forbidden"],
                        top_k=sampling.get("top_k"), top_p=sampling.get("top_p"))

  @torch.no_grad()
  def _decode_step(self, running: List[_Seq], sampling: Dict[str, Any]) -> Tuple[torch.Tensor, torch.Tensor]:
    n = len(running)
    bucket = self._bucket(n)
    st = self._static_buffers(bucket)
    ps = self.cfg.page_size
    tok = np.zeros((bucket, 1), np.int64)
    pos = np.zeros((bucket, 1), np.int64)
    slots = np.full((bucket,), -1, np.int64)
    bt = np.zeros((bucket, self.max_blocks), np.int32)
    lens = np.zeros((bucket,), np.int32)
    for i, s in enumerate(running):
      tok[i, 0], pos[i, 0] = s.last_token, s.length
      slots[i] = s.pages[s.length // ps] * ps + s.length % ps
      bt[i, :len(s.pages)] = s.pages
      lens[i] = s.length + 1
    for name, arr in (("tokens", tok), ("positions", pos), ("slots", slots), ("block_tables", bt), ("seq_lens", lens)):
      st[name].copy_(torch.from_numpy(arr), non_blocking=True)
    # everything a captured launch bakes in by value; the forbidden ids live in an engine-owned static buffer
    key = (bucket, sampling["greedy"], sampling["temperature"], sampling["seed"], sampling["n_forbidden"],
           sampling.get("top_k"), sampling.get("top_p"))
    use_graph = self.cfg.use_cuda_graphs and self.device.type == "cuda"
    if not use_graph:
      out = self._decode_body(st, sampling)
    else:
      entry = self._graphs.pop(key, None)
      if entry is None:
        entry = self._capture(st, sampling)
        while len(self._graphs) >= self._max_graphs:      # least recently used first (dicts keep insertion order)
          self._graphs.pop(next(iter(self._graphs)))
      self._graphs[key] = entry                            # (re)insert as most recent
      if entry is False:                       # capture failed once: stay eager for this key
        out = self._decode_body(st, sampling)
      else:
        entry[0].replay()
        out = entry[1]
    self._step_counter += 1
    for s in running:
      s.length += 1
    return out[0][:n], out[1][:n]

  def _capture(self, st, sampling):
    try:
      stream = torch.cuda.Stream(device=self.device)
      stream.wait_stream(torch.cuda.current_stream(self.device))
      with torch.cuda.stream(stream):
        for _ in range(2):                     # warm-up: lazy initialisation must not be captured
          self._decode_body(st, sampling)
      torch.cuda.current_stream(self.device).wait_stream(stream)
      torch.cuda.synchronize(self.device)
      g = torch.cuda.CUDAGraph()
      with torch.cuda.graph(g):
        out = self._decode_body(st, sampling)
      return g, out
    except Exception as e:   # a model feature that cannot be captured (host sync in MoE routing, ...)
      import logging
      logging.warning("CUDA graph capture of the decode step failed (%s); running it eagerly", e)
      torch.cuda.synchronize(self.device)
      return False

  # ---- scheduler -----------------------------------------------------------------------------
  def _admit(self, waiting: Deque[_Seq], running: List[_Seq]) -> List[List[_Seq]]:
    """Moves requests from `waiting` to `running` while batch slots and pages last. Returns the
    admitted sequences grouped by identical prompt (a group is prefilled once)."""
    groups: Dict[Tuple[int, ...], List[_Seq]] = {}
    alloc = self.cache.allocator
    ps = self.cfg.page_size
    while waiting and len(running) < self.cfg.max_batch:
      s = waiting[0]
      if len(s.prompt) + s.max_new > self.cfg.max_seq_len:
        raise ValueError(f"request of {len(s.prompt)} prompt + {s.max_new} new tokens exceeds max_seq_len "
                         f"{self.cfg.max_seq_len}")
      leader = groups.get(s.prompt, [None])[0] if self.cfg.share_prefix else None
      full = len(s.prompt) // ps if leader is not None else 0       # prompt pages that can be shared
      need = self._pages_needed(s) - full
      if need > alloc.free_pages:
        break
      waiting.popleft()
      s.pages = (alloc.share(leader.pages[:full]) if full else []) + alloc.alloc(need)
      groups.setdefault(s.prompt, []).append(s)
      running.append(s)
    return list(groups.values())

  def _prefill_groups(self, groups: List[List[_Seq]], sampling, results) -> None:
    """Prefills one representative per group, batching equal lengths under the token budget;
    followers copy the representative's partial tail page; all sample their first token."""
    if not groups:
      return
    ps = self.cfg.page_size
    by_len: Dict[int, List[List[_Seq]]] = {}
    for g in groups:
      by_len.setdefault(len(g[0].prompt), []).append(g)
    for L, gs in by_len.items():
      per = max(1, self.cfg.max_prefill_tokens // max(L, 1))
      for i in range(0, len(gs), per):
        chunk = gs[i:i + per]
        leaders = [g[0] for g in chunk] if self.cfg.share_prefix else [s for g in chunk for s in g]
        logits = self._prefill(leaders)
        rows = []
        for li, g in enumerate(chunk):
          members = g if self.cfg.share_prefix else []
          for s in members[1:]:
            tail = L % ps
            if tail:
              self.cache.copy_page(g[0].pages[L // ps], s.pages[L // ps], tail)
            s.length = L
          rows += [li] * len(g) if self.cfg.share_prefix else []
        if self.cfg.share_prefix:
          seqs = [s for g in chunk for s in g]
          logits = logits[torch.tensor(rows, device=logits.device)]
        else:
          seqs = leaders
        tok, lp = self._sample(logits.contiguous(), sampling)
        self._step_counter += 1
        self._append(seqs, tok, lp, sampling, results)

  def _append(self, seqs: List[_Seq], tok: torch.Tensor, lp: Optional[torch.Tensor], sampling, results) -> None:
    toks = tok.tolist()
    lps = lp.tolist() if lp is not None else [0.0] * len(toks)
    eos = sampling["eos"]
    for s, t, l in zip(seqs, toks, lps):
      s.out.append(t)
      s.lps.append(l)
      s.last_token = t
      if t in eos:
        s.reason = "eos"
      elif len(s.out) >= s.max_new:
        s.reason = "length"

  def _retire(self, running: List[_Seq], results: Dict[int, _Seq]) -> List[_Seq]:
    keep = []
    for s in running:
      if s.reason:
        self.cache.allocator.free(s.pages)
        s.pages = []
        results[s.rid] = s
      else:
        keep.append(s)
    return keep

  @torch.no_grad()
  def generate(self, prompts: Sequence[Sequence[int]], max_new_tokens: int, *, temperature: float = 1.0,
               greedy: bool = False, seed: int = 0, eos_ids: Sequence[int] = (), forbidden: Sequence[int] = (),
               return_logprobs: bool = True, top_k: Optional[int] = None,
               top_p: Optional[float] = None) -> GenerationResult:
    """Generates up to `max_new_tokens` per prompt (token id lists, unpadded). `top_k` / `top_p` restrict
    the candidates as the dense sampler does (top-p over the top-k sorted distribution)."""
    was_training = self.model.training
    self.model.eval()
    from ..ops import functional as F
    old_bound = F.set_position_bound(self.cfg.max_seq_len)
    forbidden = [int(f) for f in forbidden]
    if len(forbidden) > self._max_forbidden:
      raise ValueError(f"at most {self._max_forbidden} forbidden token ids are supported, got {len(forbidden)}")
    if forbidden:     # captured graphs read this buffer: rewrite it in place, never reallocate it
      self._forbidden[:len(forbidden)].copy_(torch.tensor(forbidden, dtype=torch.int32))
    sampling = {"temperature": float(temperature), "greedy": bool(greedy or temperature == 0.0), "seed": int(seed),
                "eos": set(int(e) for e in eos_ids), "top_k": top_k, "top_p": top_p,
                "n_forbidden": len(forbidden)}
    self._step_counter.zero_()
    waiting: Deque[_Seq] = deque(_Seq(i, tuple(int(t) for t in p), int(max_new_tokens)) for i, p in enumerate(prompts))
    for s in waiting:
      if not s.prompt:
        raise ValueError("empty prompt")
    running: List[_Seq] = []
    results: Dict[int, _Seq] = {}
    steps = 0
    timed = self.device.type == "cuda"
    prefill_marks = []
    try:
      while waiting or running:
        groups = self._admit(waiting, running)
        if not groups and not running:
          raise OutOfPages(f"a request needs {self._pages_needed(waiting[0])} pages but the cache has only "
                           f"{self.cache.num_pages}")
        if groups and timed:
          marks = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
          marks[0].record()
          self._prefill_groups(groups, sampling, results)
          marks[1].record()
          prefill_marks.append(marks)
        else:
          self._prefill_groups(groups, sampling, results)
        running = self._retire(running, results)
        if not running:
          continue
        tok, lp = self._decode_step(running, sampling)
        steps += 1
        self._append(running, tok, lp, sampling, results)
        running = self._retire(running, results)
    finally:
      for s in running:                      # only on an error path
        self.cache.allocator.free(s.pages)
      self.model.train(was_training)
      F.set_position_bound(old_bound)
    if self.device.type == "cuda":
      from ..ops import _lib
      _lib.check_status(self.device)     # a kernel that gave up a bounded wait or met a bad argument: not a result
    order = [results[i] for i in range(len(prompts))]
    prefill_ms = 0.0
    if prefill_marks:
      prefill_marks[-1][1].synchronize()
      prefill_ms = float(sum(a.elapsed_time(b) for a, b in prefill_marks))
    return GenerationResult(prefill_ms=prefill_ms, tokens=[np.asarray(s.out, dtype=np.int64) for s in order],
                            logprobs=[np.asarray(s.lps, dtype=np.float32) for s in order] if return_logprobs else None,
                            finish_reasons=[s.reason for s in order], steps=steps)
