"""RL utilities: weight-sharing checks, batch slicing / merging, critic construction, un-padding
and streaming first-fit-decreasing sequence packing (tunix/rl/utils.py:43-748)."""
from __future__ import annotations

import copy
import dataclasses
import logging
from itertools import chain
from typing import Any, Dict, Iterator, List, Mapping, Optional, Sequence, Tuple

import numpy as np
import torch

from . import common

log = logging.getLogger(__name__)


def is_positive_integer(value: Optional[int], name: str):
  if value is None:
    return
  if isinstance(value, bool) or not isinstance(value, (int, np.integer)):
    raise ValueError(f"{name} must be a positive integer. Got: {value}")
  if value <= 0:
    raise ValueError(f"{name} must be a positive integer. Got: {value}")


def check_divisibility(small_size, big_size, small_size_name, big_size_name):
  if big_size % small_size != 0:
    raise ValueError(f"{big_size_name} must be a multiple of {small_size_name}.")


def _params(m, lora: Optional[bool] = None):
  return [p for p in m.parameters() if lora is None or bool(getattr(p, "is_lora", False)) == lora]


def is_sharing_weights(m1: Optional[torch.nn.Module], m2: Optional[torch.nn.Module]) -> bool:
  """True when both modules hold the very same parameter storages."""
  if m1 is None or m2 is None:
    return False
  p1, p2 = _params(m1), _params(m2)
  return len(p1) == len(p2) and all(a.data_ptr() == b.data_ptr() for a, b in zip(p1, p2))


def is_sharing_backbone(m1: torch.nn.Module, m2: torch.nn.Module) -> bool:
  """Same as `is_sharing_weights` but ignoring LoRA adapter parameters."""
  p1, p2 = _params(m1, False), _params(m2, False)
  return len(p1) == len(p2) and all(a.data_ptr() == b.data_ptr() for a, b in zip(p1, p2))


def chunk_slices_by_size(stop: int, step: int):
  i = 0
  while i < stop:
    yield slice(i, min(i + step, stop))
    i += step


def get_batch_slice(tree: Any, batch_slice: slice) -> Any:
  """Slices array leaves (ndim >= 1) of a dict / dataclass / list batch along axis 0."""
  def rec(x):
    if x is None:
      return None
    if dataclasses.is_dataclass(x) and not isinstance(x, type):
      return dataclasses.replace(x, **{f.name: rec(getattr(x, f.name)) for f in dataclasses.fields(x)
                                       if f.name != "num_segments"})
    if isinstance(x, dict):
      return {k: rec(v) for k, v in x.items()}
    if isinstance(x, list):
      return x[batch_slice]
    if hasattr(x, "ndim") and hasattr(x, "shape") and x.ndim >= 1:
      return x[batch_slice]
    return x
  return rec(tree)


def merge_micro_batches(batches: Sequence[Mapping[str, Any]]) -> Dict[str, Any]:
  """Concatenates micro-batch dicts along the batch dimension (lists are chained)."""
  if not batches:
    return {}
  merged = {}
  for key in batches[0].keys():
    vals = [b[key] for b in batches]
    if isinstance(vals[0], list):
      merged[key] = list(chain.from_iterable(vals))
    elif isinstance(vals[0], torch.Tensor):
      merged[key] = torch.cat([v.reshape(-1) if v.dim() == 0 else v for v in vals])
    else:
      merged[key] = np.concatenate([np.atleast_1d(v) for v in vals])
  return merged


class ScoreHead(torch.nn.Module):
  """Linear(D -> 1) without bias, the value / reward head."""

  def __init__(self, dim: int, dtype=None, device=None, seed: int = 0):
    super().__init__()
    g = torch.Generator().manual_seed(seed)
    w = torch.empty(1, dim).normal_(0.0, 0.02, generator=g)
    self.w = torch.nn.Parameter(w.to(dtype=dtype or torch.float32, device=device))

  def forward(self, h):
    return torch.nn.functional.linear(h.to(self.w.dtype), self.w)


class TransformerWithScoreHead(torch.nn.Module):
  """A decoder whose output is a per-token scalar: last hidden state -> Linear(D, 1)."""

  def __init__(self, transformer: torch.nn.Module, seed: int = 0):
    super().__init__()
    cfg = getattr(transformer, "config", None)
    dim = getattr(transformer, "embed_dim", None) or getattr(cfg, "embed_dim", None)
    if dim is None:
      raise ValueError("Could not determine embed dim for the transformer.")
    self.transformer = transformer
    p = next(transformer.parameters())
    self.score = ScoreHead(dim, p.dtype, p.device, seed)
    self.config = cfg

  def forward(self, input_tokens, positions=None, cache=None, attention_mask=None, **kwargs):
    kwargs.pop("skip_lm_head", None)
    hidden, new_cache = self.transformer(input_tokens, positions, cache, attention_mask, skip_lm_head=True, **kwargs)
    return self.score(hidden), new_cache


def create_critic_model(actor_model: torch.nn.Module, seed: int = 0, lm_head_to_replace: str = "lm_head"):
  """A deep copy of the actor whose output head is replaced by Linear(D -> 1)."""
  del lm_head_to_replace
  return TransformerWithScoreHead(copy.deepcopy(actor_model), seed)


def put_params_on_memory_kind(model: torch.nn.Module, memory_kind: str) -> None:
  """Moves parameters between device memory ("device") and pinned host memory ("pinned_host")."""
  for p in model.parameters():
    if memory_kind == "pinned_host":
      if p.device.type != "cpu":
        p._home_device = p.device
        host = torch.empty(p.shape, dtype=p.dtype, device="cpu", pin_memory=torch.cuda.is_available())
        host.copy_(p.data, non_blocking=True)
        p.data = host
    elif memory_kind == "device":
      home = getattr(p, "_home_device", None)
      if home is not None and p.device != home:
        p.data = p.data.to(home, non_blocking=True)
    else:
      raise ValueError(f"unknown memory kind {memory_kind!r}")
  if torch.cuda.is_available():
    torch.cuda.synchronize()


def _np(x):
  if x is None:
    return None
  if isinstance(x, torch.Tensor):
    return x.detach().cpu().numpy()
  return np.asarray(x)


def unpad_train_example(example) -> List[Dict[str, Any]]:
  """Splits a padded batch into per-sequence dicts (prompts are left-padded, completions right-padded)."""
  res = []
  p_ids, p_mask = _np(example.prompt_ids), _np(example.prompt_mask)
  c_ids, c_mask = _np(example.completion_ids), _np(example.completion_mask)
  adv = _np(example.advantages)
  per_tok = adv.ndim == 2
  opt = {k: _np(getattr(example, k, None)) for k in ("ref_per_token_logps", "old_per_token_logps", "returns",
                                                      "old_values", "policy_version", "sampler_is_weights")}
  for i in range(p_ids.shape[0]):
    pl, cl = int(p_mask[i].sum()), int(c_mask[i].sum())
    item = {
        "prompt_ids": p_ids[i, -pl:] if pl > 0 else p_ids[i, :0],
        "prompt_mask": p_mask[i, -pl:] if pl > 0 else p_mask[i, :0],
        "completion_ids": c_ids[i, :cl],
        "completion_mask": c_mask[i, :cl],
        "advantages": adv[i, :cl] if per_tok else adv[i],
        "adv_is_per_token": per_tok,
    }
    for k, v in opt.items():
      if k == "policy_version":
        item[k] = v[i:i + 1] if v is not None else None
      else:
        item[k] = v[i, :cl] if v is not None else None
    res.append(item)
  return res


def compute_pack_size(mesh) -> int:
  """Packed rows per batch = product of the "fsdp" / "dp" mesh axes (1 without a mesh)."""
  if mesh is None:
    return 1
  return mesh.axis_size("fsdp") * mesh.axis_size("dp")


def validate_packing_budget(max_token_budget: int, max_prompt_length: int, max_response_length: int) -> None:
  longest = max_prompt_length + max_response_length
  if max_token_budget < longest:
    raise ValueError(f"max_seq_token_per_tpu={max_token_budget} is smaller than the longest possible sequence "
                     f"(max_prompt_length {max_prompt_length} + max_response_length {max_response_length} = "
                     f"{longest}); packing would fail once a maximal sequence appears. Set max_seq_token_per_tpu >= "
                     f"{longest}.")


def _item_tokens(item: Mapping[str, Any]) -> int:
  return len(item["prompt_ids"]) + len(item["completion_ids"])


def _fill_one_chunk(items, pack_size: int, budget: int, max_segments: int):
  """First-fit-decreasing into `pack_size` bins bounded by tokens and by segment count.
  Returns (bins, leftover in original order). Uses the native packer when it is built."""
  lengths = [_item_tokens(it) for it in items]
  assign = None
  try:
    from ..runtime import native
    assign = native.ffd_pack(lengths, pack_size, budget, max_segments)
  except Exception:
    assign = None
  bins: List[List[Any]] = [[] for _ in range(pack_size)]
  leftover: List[Any] = []
  if assign is None:
    loads = [0] * pack_size
    order = sorted(range(len(items)), key=lambda i: lengths[i], reverse=True)
    placed = {}
    for i in order:
      for b in range(pack_size):
        if loads[b] + lengths[i] <= budget and len(bins[b]) < max_segments:
          bins[b].append(items[i])
          loads[b] += lengths[i]
          placed[i] = b
          break
    leftover = [items[i] for i in sorted(set(range(len(items))) - set(placed), key=lambda i: (-lengths[i], i))]
  else:
    order = sorted(range(len(items)), key=lambda i: lengths[i], reverse=True)
    for i in order:
      if assign[i] >= 0:
        bins[assign[i]].append(items[i])
      else:
        leftover.append(items[i])
  return bins, leftover


_TRACKED = ("ref_per_token_logps", "old_per_token_logps", "returns", "old_values", "sampler_is_weights")


def pack_sequences(item_iterator: Iterator[Sequence[Any]], max_token_budget: int, sequences_per_update: int,
                   pad_id: int = 0, pack_size: int = 1,
                   max_segments_per_packed_row: Optional[int] = None) -> Iterator[List[Any]]:
  """Streams `[pack_size, max_token_budget]` packed examples out of a stream of padded batches.

  Each packed row holds whole sequences (prompt then completion) with `segment_ids` 1..K and
  per-segment positions; padding is segment 0. A chunk is emitted as soon as the buffered
  sequences fill it; the last chunk of every `sequences_per_update` sequences carries
  `is_update_step=True`. Errors: empty mini-batch at a boundary, a sequence longer than the
  budget, a stream ending mid mini-batch, or a boundary inside an input example."""
  max_seg = max_segments_per_packed_row if max_segments_per_packed_row is not None else max_token_budget
  state = {"cls": common.TrainExample, "first": None}

  def flush_row(row_items) -> Dict[str, np.ndarray]:
    first = state["first"] or {}
    tracked = [k for k in _TRACKED if first.get(k) is not None]
    B = max_token_budget
    out = {"completion_ids": np.full(B, pad_id, np.int64), "completion_mask": np.zeros(B, np.int32),
           "advantages": np.zeros(B, np.float32), "segment_ids": np.zeros(B, np.int32),
           "segment_positions": np.zeros(B, np.int32)}
    for k in tracked:
      out[k] = np.zeros(B, np.float32)
    if len(row_items) > max_seg:
      raise ValueError(f"pack_sequences: a packed row has {len(row_items)} segments, exceeding "
                       f"max_segments_per_packed_row={max_seg}; increase it (or leave it None for the "
                       "budget-derived safe default).")
    o = 0
    for s, it in enumerate(row_items, start=1):
      pl, cl = len(it["prompt_ids"]), len(it["completion_ids"])
      n = pl + cl
      out["completion_ids"][o:o + pl] = it["prompt_ids"]
      out["completion_ids"][o + pl:o + n] = it["completion_ids"]
      out["completion_mask"][o + pl:o + n] = it["completion_mask"]
      out["advantages"][o + pl:o + n] = it["advantages"]
      for k in tracked:
        out[k][o + pl:o + n] = it[k]
      out["segment_ids"][o:o + n] = s
      out["segment_positions"][o:o + n] = np.arange(n)
      o += n
    return out

  def emit(chunk, is_update: bool):
    rows = [flush_row(r) for r in chunk]
    stack = {k: torch.from_numpy(np.stack([r[k] for r in rows])) for k in rows[0]}
    n = len(rows)
    kwargs = dict(prompt_ids=torch.zeros(n, 0, dtype=torch.long), prompt_mask=torch.zeros(n, 0, dtype=torch.int32),
                  completion_ids=stack["completion_ids"], completion_mask=stack["completion_mask"],
                  advantages=stack["advantages"], ref_per_token_logps=stack.get("ref_per_token_logps"),
                  old_per_token_logps=stack.get("old_per_token_logps"), segment_ids=stack["segment_ids"],
                  segment_positions=stack["segment_positions"], num_segments=max_seg + 1,
                  is_update_step=torch.tensor([is_update]))
    cls = state["cls"]
    names = {f.name for f in dataclasses.fields(cls)}
    for k in ("returns", "old_values", "sampler_is_weights"):
      if k in names and k in stack:
        kwargs[k] = stack[k]
    first = state["first"] or {}
    if "policy_version" in names and first.get("policy_version") is not None:
      kwargs["policy_version"] = torch.as_tensor(first["policy_version"])
    return [cls(**{k: v for k, v in kwargs.items() if k in names})]

  cap = pack_size * max_token_budget
  buffered: List[Dict[str, Any]] = []
  received = tokens = chunks = 0

  def final_flush():
    nonlocal buffered, received, tokens, chunks
    if not buffered and chunks == 0:
      raise ValueError("pack_sequences reached an update boundary with an empty mini-batch; no packed example "
                       "would be produced, dropping a gradient update.")
    while buffered:
      chunk, buffered = _fill_one_chunk(buffered, pack_size, max_token_budget, max_seg)
      chunks += 1
      yield emit(chunk, not buffered)
    total = chunks * cap
    log.info("pack_sequences: %d seqs -> %d chunks, dummy_ratio=%.3f", received, chunks,
             1.0 - tokens / total if total else 0.0)
    received = tokens = chunks = 0

  for item_list in item_iterator:
    for example in item_list:
      state["cls"] = type(example)
      for item in unpad_train_example(example):
        n = _item_tokens(item)
        if n > max_token_budget:
          raise ValueError(f"pack_sequences: a single sequence has {n} tokens, exceeding max_token_budget "
                           f"{max_token_budget}; increase the budget.")
        if state["first"] is None:
          state["first"] = item
        if not item["adv_is_per_token"]:
          item["advantages"] = np.full(len(item["completion_ids"]), item["advantages"], dtype=np.float32)
        buffered.append(item)
        received += 1
        tokens += n
    if received > sequences_per_update:
      raise ValueError("pack_sequences: mini-batch boundary falls inside an input example (received "
                       f"{received} sequences, expected {sequences_per_update} per update).")
    if received == sequences_per_update:
      yield from final_flush()
    else:
      while sum(_item_tokens(it) for it in buffered) >= cap:
        chunk, buffered = _fill_one_chunk(buffered, pack_size, max_token_budget, max_seg)
        chunks += 1
        yield emit(chunk, False)
  if buffered or received:
    raise ValueError("pack_sequences stream ended mid-mini-batch.")
