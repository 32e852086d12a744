"""Turning unbatched per-trajectory payloads into trainer micro-batches
(tunix/experimental/orchestrator/batch_assembly.py:34-600).

`GRPOTrainExampleAssembler`: left-padded prompts + right-padded completions as `TrainExample`s
(what the GRPO / PPO losses consume); short chunks are filled with all-masked rows so every
micro-batch has the same shape. `PaddedBatchAssembler`: right-padded `[B, T]` token streams.
`SequencePackedBatchAssembler`: first-fit-decreasing packing of whole sequences into rows of
`max_packed_len` with segment ids and per-segment positions.
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
  """A per-token array given either over the completion or over prompt+completion, cut to the
  kept completion tokens and right-padded to `length`."""
  out = np.full(length, fill_value, np.float32)
  if values is None:
    return out
  v = np.asarray(values, np.float32).reshape(-1)
  full = full_completion_len if full_completion_len is not None else kept
  if len(v) == prompt_len + full and prompt_len:
    v = v[prompt_len:]
  out[:min(kept, len(v))] = v[:kept]
  return out


def with_ref_per_token_logps(batch: rl_common.TrainExample, ref_logps) -> rl_common.TrainExample:
  return dataclasses.replace(batch, ref_per_token_logps=np.asarray(ref_logps, np.float32))


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
        rows["ref"].append(_completion_aligned(it.ref_per_token_logps, len(c), C, full_completion_len=len(c_full)))
      if has_old:
        rows["old"].append(_completion_aligned(it.old_per_token_logps, len(c), C, full_completion_len=len(c_full)))
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


class PaddedBatchAssembler:
  def __init__(self, batch_size: int = 8, max_len: int = 8192, pad_id: int = 0):
    self.batch_size, self.max_len, self.pad_id = batch_size, max_len, pad_id

  def pack(self, items: Sequence[datatypes.RLTrainerPayload]) -> List[datatypes.RLTrainerPayload]:
    items = list(items)
    return [self._pack_chunk(items[i:i + self.batch_size]) for i in range(0, len(items), self.batch_size)]

  def _pack_chunk(self, chunk) -> datatypes.RLTrainerPayload:
    T_ = min(self.max_len, max(len(np.asarray(x.token_ids).reshape(-1)) for x in chunk))
    def col(get, fill, dtype):
      return np.stack([_right_pad(np.asarray(get(x)).reshape(-1), T_, fill, dtype)[0] for x in chunk])
    return datatypes.RLTrainerPayload(
        token_ids=col(lambda x: x.token_ids, self.pad_id, np.int32),
        token_mask=col(lambda x: x.token_mask, 0.0, np.float32), loss_mask=col(lambda x: x.loss_mask, 0.0, np.float32),
        advantages=col(lambda x: x.advantages, 0.0, np.float32), action_mask=col(lambda x: x.loss_mask, 0.0, np.float32))


class SequencePackedBatchAssembler:
  def __init__(self, max_packed_len: int = 8192, pad_id: int = 0):
    self.max_packed_len, self.pad_id = max_packed_len, pad_id

  def pack(self, items: Sequence[datatypes.RLTrainerPayload]) -> List[datatypes.RLTrainerPayload]:
    """One packed row per output payload ([1, max_packed_len]); sequences longer than the row are
    truncated on the right."""
    L = self.max_packed_len
    seqs = sorted((x for x in items if x is not None), key=lambda x: -len(np.asarray(x.token_ids).reshape(-1)))
    bins: List[List[Any]] = []
    room: List[int] = []
    for x in seqs:
      n = min(len(np.asarray(x.token_ids).reshape(-1)), L)
      for b in range(len(bins)):
        if room[b] >= n:
          bins[b].append(x); room[b] -= n
          break
      else:
        bins.append([x]); room.append(L - n)
    out = []
    for b in bins:
      tok = np.full(L, self.pad_id, np.int32)
      mask = np.zeros(L, np.float32); loss = np.zeros(L, np.float32); adv = np.zeros(L, np.float32)
      seg = np.zeros(L, np.int32); pos = np.zeros(L, np.int32)
      off = 0
      for s, x in enumerate(b, start=1):
        t = np.asarray(x.token_ids, np.int32).reshape(-1)[:L - off]
        n = len(t)
        tok[off:off + n] = t
        mask[off:off + n] = 1.0
        loss[off:off + n] = np.asarray(x.loss_mask, np.float32).reshape(-1)[:n]
        adv[off:off + n] = np.asarray(x.advantages, np.float32).reshape(-1)[:n]
        seg[off:off + n] = s
        pos[off:off + n] = np.arange(n)
        off += n
      out.append(datatypes.RLTrainerPayload(token_ids=tok[None], token_mask=mask[None], loss_mask=loss[None],
                                            advantages=adv[None], action_mask=loss[None], segment_ids=seg[None],
                                            segment_positions=pos[None]))
    return out
