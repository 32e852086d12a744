"""Turning unbatched per-trajectory payloads into trainer micro-batches
(tunix/experimental/orchestrator/batch_assembly.py:34-600).

`GRPOTrainExampleAssembler`: left-padded prompts + right-padded completions as `TrainExample`s
(what the GRPO / PPO losses consume); short chunks are filled with all-masked rows so every
micro-batch has the same shape. `PaddedBatchAssembler`: fixed `[B, max_seq_len]` batches over whole token streams.
`SequencePackedBatchAssembler`: first-fit-decreasing packing of whole streams into rows of
`max_packed_len` with segment ids and per-segment positions. The two stream assemblers share `_StreamRow`
(truncation, action mask, scalar advantages, optional per-token fields).
"""
from __future__ import annotations

import dataclasses
from typing import Any, Generic, List, Optional, Protocol, Sequence, TypeVar

import numpy as np

from ...rl import common as rl_common
from ..common import datatypes

T = TypeVar("T")


class BatchAssembler(Generic[T], Protocol):
  def pack(self, items: Sequence[T]) -> List[Any]: ...


def _left_pad(x: np.ndarray, length: int, pad_id: int):
  x = x[-length:]
  n = length - len(x)
  return (np.concatenate([np.full(n, pad_id, x.dtype), x]),
          np.concatenate([np.zeros(n, np.float32), np.ones(len(x), np.float32)]))


def _right_pad(x: np.ndarray, length: int, pad_value, dtype):
  x = np.asarray(x, dtype=dtype)[:length]
  n = length - len(x)
  return (np.concatenate([x, np.full(n, pad_value, dtype)]),
          np.concatenate([np.ones(len(x), np.float32), np.zeros(n, np.float32)]))


def _completion_aligned(values, kept: int, length: int, fill_value: float = 0.0, prompt_len: int = 0,
                        full_completion_len: Optional[int] = None) -> np.ndarray:
  """A per-token array given either over the completion or over prompt+completion (or one scalar for the whole
  sequence), cut to the kept completion tokens and right-padded to `length`."""
  out = np.full(length, fill_value, np.float32)
  if values is None:
    return out
  if np.ndim(values) == 0:              # one value for the sequence (GRPO advantages): every kept token gets it
    out[:kept] = np.float32(values)
    return out
  v = np.asarray(values, np.float32).reshape(-1)
  full = full_completion_len if full_completion_len is not None else kept
  if len(v) == prompt_len + full and prompt_len:
    v = v[prompt_len:]
  out[:min(kept, len(v))] = v[:kept]
  return out


def with_ref_per_token_logps(batch: rl_common.TrainExample, ref_logps) -> rl_common.TrainExample:
  """The batch with reference log-probs attached. `ref_logps` is a `[B, C]` array aligned with the padded
  completions, or the `LogprobsResponse` an inference worker answered with (an error inside it is raised here,
  where the caller can still decide what to do with the batch)."""
  if not isinstance(batch, rl_common.TrainExample):
    raise TypeError(f"with_ref_per_token_logps expects a padded TrainExample from a batch assembler; got "
                    f"{type(batch).__name__}.")
  if isinstance(ref_logps, datatypes.LogprobsResponse):
    if ref_logps.error is not None:
      raise RuntimeError(ref_logps.error.message)
    ref_logps = ref_logps.per_token_logps
  values = np.asarray(ref_logps, np.float32)
  want = np.asarray(batch.completion_ids).shape
  if values.shape != want:
    raise ValueError(f"Reference logps shape must match padded completion_ids shape: got {values.shape}, expected "
                     f"{want}.")
  return dataclasses.replace(batch, ref_per_token_logps=values)


class GRPOTrainExampleAssembler:
  def __init__(self, *, batch_size: int, max_prompt_length: int, max_response_length: int, pad_id: int):
    if batch_size <= 0:
      raise ValueError("train microbatch size must be positive.")
    self.batch_size, self.pad_id = batch_size, pad_id
    self.max_prompt_length, self.max_response_length = max_prompt_length, max_response_length

  def pack(self, items: Sequence[datatypes.RLTrainerPayload]) -> List[rl_common.TrainExample]:
    items = list(items)
    return [self._pack_chunk(items[i:i + self.batch_size]) for i in range(0, len(items), self.batch_size)]

  def _pack_chunk(self, chunk) -> rl_common.TrainExample:
    P, C, pad = self.max_prompt_length, self.max_response_length, self.pad_id
    has_ref = any(x.ref_per_token_logps is not None for x in chunk)
    has_old = any(x.old_per_token_logps is not None for x in chunk)
    rows = {k: [] for k in ("p", "pm", "c", "cm", "adv", "ref", "old")}
    for it in chunk:
      p = np.asarray(it.prompt_ids, np.int32).reshape(-1)
      c_full = np.asarray(it.completion_ids, np.int32).reshape(-1)
      c = c_full[:C]
      src = (np.asarray(it.completion_mask, np.float32).reshape(-1) if it.completion_mask is not None
             else np.ones(len(c_full), np.float32))[:len(c)]
      p_ids, p_mask = _left_pad(p, P, pad)
      c_ids, _ = _right_pad(c, C, pad, np.int32)
      c_mask = np.zeros(C, np.float32)
      c_mask[:len(src)] = src
      rows["p"].append(p_ids); rows["pm"].append(p_mask); rows["c"].append(c_ids); rows["cm"].append(c_mask)
      rows["adv"].append(_completion_aligned(it.advantages, len(c), C, 0.0, len(p), len(c_full)))
      if has_ref:
        rows["ref"].append(_completion_aligned(it.ref_per_token_logps, len(c), C, 0.0, len(p), len(c_full)))
      if has_old:
        rows["old"].append(_completion_aligned(it.old_per_token_logps, len(c), C, 0.0, len(p), len(c_full)))
    while len(rows["p"]) < self.batch_size:          # all-masked filler rows keep shapes static
      rows["p"].append(np.full(P, pad, np.int32)); rows["pm"].append(np.zeros(P, np.float32))
      rows["c"].append(np.full(C, pad, np.int32)); rows["cm"].append(np.zeros(C, np.float32))
      rows["adv"].append(np.zeros(C, np.float32))
      if has_ref:
        rows["ref"].append(np.zeros(C, np.float32))
      if has_old:
        rows["old"].append(np.zeros(C, np.float32))
    # GRPO uses one advantage per sequence; per-token advantages (PPO) are kept as they are
    adv = np.stack(rows["adv"])
    cm = np.stack(rows["cm"])
    per_seq = np.array([a[m > 0][0] if (m > 0).any() else 0.0 for a, m in zip(adv, cm)], np.float32)
    uniform = all(np.allclose(a[m > 0], a[m > 0][0]) for a, m in zip(adv, cm) if (m > 0).any())
    return rl_common.TrainExample(
        prompt_ids=np.stack(rows["p"]).astype(np.int64), prompt_mask=np.stack(rows["pm"]) > 0,
        completion_ids=np.stack(rows["c"]).astype(np.int64), completion_mask=cm > 0,
        advantages=per_seq if uniform else adv,
        ref_per_token_logps=np.stack(rows["ref"]) if has_ref else None,
        old_per_token_logps=np.stack(rows["old"]) if has_old else None)


# Per-token fields a token-stream payload may carry besides the mandatory ones; each is emitted for a batch when
# at least one of its rows has it (rows without it contribute zeros, so rows stay aligned across fields).
_OPTIONAL_STREAM_FIELDS = ("ref_per_token_logps", "old_per_token_logps", "returns", "old_values", "sampler_is_weights")


def _stream(x: Any, dtype) -> np.ndarray:
  return np.asarray(x, dtype).reshape(-1)


class _StreamRow:
  """One trajectory as aligned per-token arrays over its (possibly truncated) token stream."""

  def __init__(self, item: datatypes.RLTrainerPayload, limit: int):
    self.tokens = _stream(item.token_ids, np.int32)[:limit]
    n = self.n = len(self.tokens)
    self.loss = self._fit(item.loss_mask, n)
    # the action mask marks the tokens the policy itself produced (tool observations inside a trajectory are not)
    self.action = self._fit(item.action_mask, n) if item.action_mask is not None else self.loss
    adv = item.advantages
    if adv is None:
      self.adv = np.zeros(n, np.float32)
    elif np.ndim(adv) == 0 or np.size(adv) == 1:
      self.adv = np.float32(np.asarray(adv).reshape(-1)[0]) * (self.loss > 0)      # one value per sequence
    else:
      self.adv = self._fit(adv, n)
    self.optional = {name: self._fit(getattr(item, name), n) for name in _OPTIONAL_STREAM_FIELDS
                     if getattr(item, name, None) is not None}

  @staticmethod
  def _fit(values: Any, n: int) -> np.ndarray:
    """Cut or zero-extended to n entries."""
    v = _stream(values, np.float32)[:n]
    return v if len(v) == n else np.concatenate([v, np.zeros(n - len(v), np.float32)])


class PaddedBatchAssembler:
  """Rectangular `[batch_size, max_seq_len]` payloads over whole token streams (multi-turn trajectories: prompt,
  model turns and tool observations in one row). Rows are right-padded, over-long streams cut on the right, and a
  short last chunk is filled with all-masked rows, so every micro-batch has the same shape. Only the token-stream
  fields are read: `prompt_ids` / `completion_ids` of an item play no role here."""

  def __init__(self, batch_size: int = 8, max_seq_len: Optional[int] = None, pad_id: int = 0, *,
               max_len: Optional[int] = None):
    length = max_seq_len if max_seq_len is not None else (max_len if max_len is not None else 8192)
    if batch_size <= 0:
      raise ValueError(f"batch_size must be positive, got {batch_size}.")
    if length <= 0:
      raise ValueError(f"max_seq_len must be positive, got {length}.")
    self.batch_size, self.max_seq_len, self.pad_id = int(batch_size), int(length), pad_id

  @property
  def max_len(self) -> int:
    return self.max_seq_len

  def pack(self, items: Sequence[datatypes.RLTrainerPayload]) -> List[datatypes.RLTrainerPayload]:
    rows = [_StreamRow(x, self.max_seq_len) for x in items]
    return [self._batch(rows[i:i + self.batch_size]) for i in range(0, len(rows), self.batch_size)]

  def _batch(self, rows: Sequence[_StreamRow]) -> datatypes.RLTrainerPayload:
    B, L = self.batch_size, self.max_seq_len
    tokens = np.full((B, L), self.pad_id, np.int32)
    planes = {k: np.zeros((B, L), np.float32) for k in ("token_mask", "loss_mask", "action_mask", "advantages")}
    present = [name for name in _OPTIONAL_STREAM_FIELDS if any(name in r.optional for r in rows)]
    extra = {name: np.zeros((B, L), np.float32) for name in present}
    for b, r in enumerate(rows):
      tokens[b, :r.n] = r.tokens
      planes["token_mask"][b, :r.n] = 1.0
      planes["loss_mask"][b, :r.n], planes["action_mask"][b, :r.n], planes["advantages"][b, :r.n] = r.loss, r.action, r.adv
      for name in present:
        if name in r.optional:
          extra[name][b, :r.n] = r.optional[name]
    return datatypes.RLTrainerPayload(token_ids=tokens, **planes, **extra)


class SequencePackedBatchAssembler:
  """First-fit-decreasing packing of whole token streams into rows of `max_packed_len` (one `[1, L]` payload per
  row) with segment ids 1..K and positions restarting per segment; a stream longer than a row is cut on the
  right. Optional per-token fields travel with their tokens."""

  def __init__(self, max_packed_len: int = 8192, pad_id: int = 0):
    if max_packed_len <= 0:
      raise ValueError(f"max_packed_len must be positive, got {max_packed_len}.")
    self.max_packed_len, self.pad_id = int(max_packed_len), pad_id

  def pack(self, items: Sequence[datatypes.RLTrainerPayload]) -> List[datatypes.RLTrainerPayload]:
    L = self.max_packed_len
    rows = sorted((_StreamRow(x, L) for x in items if x is not None), key=lambda r: -r.n)
    bins: List[List[_StreamRow]] = []
    room: List[int] = []
    for r in rows:
      slot = next((b for b in range(len(bins)) if room[b] >= r.n), None)
      if slot is None:
        bins.append([r])
        room.append(L - r.n)
      else:
        bins[slot].append(r)
        room[slot] -= r.n
    return [self._row(members) for members in bins]

  def _row(self, members: Sequence[_StreamRow]) -> datatypes.RLTrainerPayload:
    L = self.max_packed_len
    tokens = np.full((1, L), self.pad_id, np.int32)
    planes = {k: np.zeros((1, L), np.float32) for k in ("token_mask", "loss_mask", "action_mask", "advantages")}
    segment, position = np.zeros((1, L), np.int32), np.zeros((1, L), np.int32)
    present = [name for name in _OPTIONAL_STREAM_FIELDS if any(name in r.optional for r in members)]
    extra = {name: np.zeros((1, L), np.float32) for name in present}
    at = 0
    for k, r in enumerate(members, start=1):
      span = slice(at, at + r.n)
      tokens[0, span], segment[0, span], position[0, span] = r.tokens, k, np.arange(r.n)
      planes["token_mask"][0, span] = 1.0
      planes["loss_mask"][0, span], planes["action_mask"][0, span], planes["advantages"][0, span] = r.loss, r.action, r.adv
      for name in present:
        if name in r.optional:
          extra[name][0, span] = r.optional[name]
      at += r.n
    return datatypes.RLTrainerPayload(token_ids=tokens, segment_ids=segment, segment_positions=position, **planes,
                                      **extra)
