"""Building blocks shared by the RL learners: the `TrainExample` batch, KL estimators,
per-token log-probabilities, completion masks, padding, segment reductions and loss
aggregation. Semantics follow tunix/rl/common.py:32-1177.

Per-token log-probabilities go through `ops.functional.linear_logprob`, i.e. the same fused
lm_head + log-softmax kernels in the trainer, the reference policy and the rollout sampler, so
their numbers agree; the `[B, T, V]` logits are never materialised (the reference needs
`compute_logps_chunk_size` for that).
"""
from __future__ import annotations

import dataclasses
import inspect
from typing import Any, Dict, Iterable, List, Optional, Tuple

import numpy as np
import torch

from ..ops import functional as F
from ..sft import utils
from ..sft.utils import build_positions_from_mask, make_causal_attn_mask

WeightedMetric = utils.WeightedMetric


def _tree_leaves(x) -> List[Any]:
  if dataclasses.is_dataclass(x) and not isinstance(x, type):
    return [l for f in dataclasses.fields(x) for l in _tree_leaves(getattr(x, f.name))]
  if isinstance(x, dict):
    return [l for v in x.values() for l in _tree_leaves(v)]
  if isinstance(x, (list, tuple)):
    return [l for v in x for l in _tree_leaves(v)]
  return [x] if isinstance(x, (torch.Tensor, np.ndarray)) else []


def tree_index(x, idx):
  """Indexes every array leaf of a batch along its leading axis."""
  if dataclasses.is_dataclass(x) and not isinstance(x, type):
    return dataclasses.replace(x, **{f.name: tree_index(getattr(x, f.name), idx) for f in dataclasses.fields(x)})
  if isinstance(x, dict):
    return {k: tree_index(v, idx) for k, v in x.items()}
  if isinstance(x, (list, tuple)):
    return type(x)(tree_index(v, idx) for v in x)
  if isinstance(x, torch.Tensor):
    return x[torch.as_tensor(idx, device=x.device)] if x.dim() > 0 else x
  if isinstance(x, np.ndarray):
    return x[np.asarray(idx)] if x.ndim > 0 else x
  return x


class RepeatIterable:
  """Iterates a list of rollout batches `repeat` times; each batch is optionally shuffled and
  cut into mini-batches."""

  def __init__(self, data: List[Any], repeat: int, mini_batch_size: Optional[int] = None, shuffle: bool = False,
               key: Any = None):
    self._data = data
    self.repeat = repeat
    self.mini_batch_size = mini_batch_size
    self.shuffle = shuffle
    seed = int(key) if key is not None and not isinstance(key, torch.Generator) else 0
    self.key = key if isinstance(key, torch.Generator) else torch.Generator().manual_seed(seed)
    self._mini_batch_size = mini_batch_size

  def _shuffle_and_slice_one_batch(self, rollout_batch: Any):
    leaves = _tree_leaves(rollout_batch)
    n = leaves[0].shape[0]
    if self.mini_batch_size is None:
      self._mini_batch_size = n
    if n % self._mini_batch_size != 0:
      raise ValueError("Each rollout batch's size must be divisible by `mini_batch_size`.")
    order = torch.randperm(n, generator=self.key) if self.shuffle else torch.arange(n)
    for i in range(n // self._mini_batch_size):
      yield tree_index(rollout_batch, order[i * self._mini_batch_size:(i + 1) * self._mini_batch_size])

  def __iter__(self):
    for _ in range(self.repeat):
      for rollout_batch in self._data:
        yield from self._shuffle_and_slice_one_batch(rollout_batch)


@dataclasses.dataclass(frozen=True)
class TrainExample:
  """One RL training micro-batch. `num_segments` is the static bound on segments per packed
  row (padding bucket 0 included); `sampler_is_weights` are detached truncated
  importance-sampling weights multiplied into the policy-gradient loss before aggregation."""

  prompt_ids: Any
  prompt_mask: Any
  completion_ids: Any
  completion_mask: Any
  advantages: Any
  ref_per_token_logps: Any
  old_per_token_logps: Any
  segment_ids: Any = None
  segment_positions: Any = None
  num_segments: Optional[int] = None
  is_update_step: Any = None
  sampler_is_weights: Any = None

  def to_tensors(self, device=None) -> "TrainExample":
    def cv(x):
      if isinstance(x, np.ndarray):
        x = torch.from_numpy(x)
      if isinstance(x, torch.Tensor) and device is not None:
        x = x.to(device)
      return x
    return dataclasses.replace(self, **{f.name: cv(getattr(self, f.name)) for f in dataclasses.fields(self)
                                        if f.name != "num_segments"})

  to_jax_array = to_tensors   # name used by code written against the reference


def compute_kl_divergence(per_token_logps: torch.Tensor, ref_per_token_logps: torch.Tensor,
                          method: str = "low_var_kl", clamp_value: Optional[float] = None) -> torch.Tensor:
  """Per-token KL between the trained and the reference policy.

  "kl": `logp - ref`; "mse_kl": `0.5 (logp - ref)^2`; "low_var_kl": `(r - 1) - log r` with
  `r = exp(ref - logp)`. `clamp_value` symmetrically clips the result."""
  lp = per_token_logps.float()
  ref = ref_per_token_logps.float() if ref_per_token_logps is not None else None
  if method == "kl":
    kl = lp - ref
  elif method == "mse_kl":
    kl = 0.5 * (lp - ref) ** 2
  elif method == "low_var_kl":
    diff = ref - lp
    kl = torch.exp(diff) - diff - 1
  else:
    raise ValueError(f"`method` must be one of 'kl', 'mse_kl', 'low_var_kl'. Received: {method}")
  if clamp_value is not None:
    kl = torch.clamp(kl, -clamp_value, clamp_value)
  return kl


def selective_log_softmax(logits: torch.Tensor, input_ids: torch.Tensor) -> torch.Tensor:
  """`logit[id] - logsumexp(logits)` in fp32."""
  lp, _ = F.ref.selective_log_softmax(logits, input_ids)
  return lp


def compute_entropy_from_logits(logits: torch.Tensor) -> torch.Tensor:
  lsm = torch.log_softmax(logits.float(), dim=-1)
  return -(lsm.exp() * lsm).sum(-1)


def process_ids(prompt_tokens: torch.Tensor, completion_tokens: torch.Tensor, pad_id: int, eos_id: int,
                segment_ids: Optional[torch.Tensor] = None, segment_positions: Optional[torch.Tensor] = None):
  """-> (prompt|completion ids, positions, attention mask or None, input segment ids or None)."""
  ids = torch.cat([prompt_tokens, completion_tokens], dim=1)
  if segment_ids is not None:
    if segment_positions is None:
      raise ValueError("segment_positions must be explicitly provided for packed sequences. ")
    return ids, segment_positions, None, None
  mask = torch.cat([prompt_tokens != pad_id, completion_tokens != pad_id], dim=-1)
  return ids, build_positions_from_mask(mask), make_causal_attn_mask(mask), mask.to(torch.int32)


def model_call_contains(model, target_arg: str) -> bool:
  target = model.transformer if hasattr(model, "transformer") else model
  try:
    sig = inspect.signature(target.forward if hasattr(target, "forward") else target.__call__)
  except (TypeError, ValueError):
    return False
  return target_arg in sig.parameters or any(p.kind == inspect.Parameter.VAR_KEYWORD for p in sig.parameters.values())


def get_per_token_logps(model, input_tokens, positions, attn_mask, logits_to_keep: int, images=None):
  """Log-probabilities of the last `logits_to_keep` tokens."""
  kwargs = {} if images is None else {"images": images}
  if hasattr(model, "head_weight"):
    hidden, _ = model(input_tokens, positions, None, attn_mask, skip_lm_head=True, **kwargs)
    h = hidden[:, -logits_to_keep - 1:-1]
    lp, _ = F.linear_logprob(h, model.head_weight(), input_tokens[:, -logits_to_keep:],
                             softcap=getattr(model.config, "final_logit_softcap", None) or 0.0)
    return lp
  logits, _ = model(input_tokens, positions, None, attn_mask, **kwargs)
  return selective_log_softmax(logits[:, -logits_to_keep - 1:-1], input_tokens[:, -logits_to_keep:])


def compute_per_token_logps(model, prompt_tokens: torch.Tensor, completion_tokens: torch.Tensor, pad_id: int,
                            eos_id: int, images=None, stop_gradient: bool = True, return_entropy: bool = False,
                            segment_ids=None, segment_positions=None, temperature: float = 1.0, chunk_size: int = 0):
  """Per-token log-probabilities (and optionally entropies) of the completion tokens.

  Unpacked: result `[B, completion_len]`. Packed (`segment_ids` given, prompts already inside
  `completion_tokens`): result `[B, full_len]`, left-padded with one 0 so position t holds the
  log-probability of token t. Logits are divided by `temperature` unless it is 0 or 1.
  `chunk_size` is accepted for compatibility; the fused kernel always works in chunks."""
  del chunk_size
  ids, positions, attn_mask, input_seg = process_ids(prompt_tokens, completion_tokens, pad_id, eos_id, segment_ids,
                                                     segment_positions)
  kwargs: Dict[str, Any] = {}
  if model_call_contains(model, "segment_ids") and segment_ids is not None:
    kwargs["segment_ids"] = segment_ids
  if images is not None:
    kwargs["images"] = images
  keep = ids.shape[1] - 1 if segment_ids is not None else completion_tokens.shape[1]
  targets = ids[:, -keep:]
  ctx = torch.no_grad() if stop_gradient else _nullcontext()
  with ctx:
    if hasattr(model, "head_weight"):
      hidden, _ = model(ids, positions, None, attn_mask, skip_lm_head=True, **kwargs)
      h = hidden[:, -keep - 1:-1]
      lp, ent = F.linear_logprob(h, model.head_weight(), targets, temperature=temperature,
                                 softcap=getattr(model.config, "final_logit_softcap", None) or 0.0,
                                 want_entropy=return_entropy)
    else:
      logits, _ = model(ids, positions, None, attn_mask, **kwargs)
      logits = logits[:, -keep - 1:-1]
      lp, ent = F.ref.selective_log_softmax(logits, targets, temperature, return_entropy)
  if segment_ids is not None:
    lp = torch.nn.functional.pad(lp, (1, 0))
    if ent is not None:
      ent = torch.nn.functional.pad(ent, (1, 0))
  if stop_gradient:
    lp = lp.detach()
    ent = ent.detach() if ent is not None else None
  return (lp, ent) if return_entropy else lp


class _nullcontext:
  def __enter__(self):
    return None

  def __exit__(self, *a):
    return False


def compute_score(model, prompt_tokens, completion_tokens, pad_id: int, eos_id: int, stop_gradient: bool = True,
                  segment_ids=None, segment_positions=None) -> torch.Tensor:
  """Per-token scalar scores of a reward / value model (last dim 1 squeezed)."""
  ids, positions, attn_mask, input_seg = process_ids(prompt_tokens, completion_tokens, pad_id, eos_id, segment_ids,
                                                     segment_positions)
  kwargs: Dict[str, Any] = {}
  if model_call_contains(model, "segment_ids") and segment_ids is not None:
    kwargs["segment_ids"] = segment_ids
  ctx = torch.no_grad() if stop_gradient else _nullcontext()
  with ctx:
    out = model(ids, positions, None, attn_mask, **kwargs)
  scores = out[0] if isinstance(out, tuple) else out
  scores = scores.squeeze(-1)
  return scores.detach() if stop_gradient else scores


def np_make_completion_mask(completion_ids: np.ndarray, eos_tok: int = 0) -> np.ndarray:
  is_eos = completion_ids == eos_tok
  L = is_eos.shape[1]
  eos_idx = np.where(np.any(is_eos, axis=1), np.argmax(is_eos, axis=1), L)
  return (np.arange(L) < eos_idx[:, None] + 1).astype(np.int32)


def make_completion_mask(completion_ids: torch.Tensor, eos_tok: int = 0) -> torch.Tensor:
  """1 up to and including the first EOS, 0 after."""
  is_eos = completion_ids == eos_tok
  L = is_eos.shape[1]
  first = torch.where(is_eos.any(dim=1), is_eos.int().argmax(dim=1), torch.full_like(is_eos[:, 0], L, dtype=torch.long))
  return (torch.arange(L, device=completion_ids.device)[None, :] <= first[:, None]).to(torch.int32)


def pad_to_length(x, target_length: int, pad_value=0, left: bool = False, axis: int = 0):
  """Pads a tensor / ndarray along `axis` up to `target_length` (no-op when already longer)."""
  is_np = isinstance(x, np.ndarray)
  length = x.shape[axis]
  if length >= target_length:
    return x
  shape = list(x.shape)
  shape[axis] = target_length - length
  if is_np:
    pad = np.full(shape, pad_value, dtype=x.dtype)
    return np.concatenate([pad, x] if left else [x, pad], axis=axis)
  pad = torch.full(shape, pad_value, dtype=x.dtype, device=x.device)
  return torch.cat([pad, x] if left else [x, pad], dim=axis)


def segmented_sum(values: torch.Tensor, segment_ids: torch.Tensor, num_segments: int) -> torch.Tensor:
  """Per-row segment sums: `[B, T]` values grouped by `[B, T]` ids -> `[B, S]`; ids >= S are dropped."""
  B = values.shape[0]
  out = torch.zeros(B, num_segments, dtype=values.dtype, device=values.device)
  ids = segment_ids.long()
  valid = (ids >= 0) & (ids < num_segments)
  return out.scatter_add(1, ids.clamp(0, num_segments - 1), values * valid.to(values.dtype))


def segmented_count(segment_ids: torch.Tensor, num_segments: int, mask: Optional[torch.Tensor] = None) -> torch.Tensor:
  ones = torch.ones_like(segment_ids, dtype=torch.float32) if mask is None else mask.float()
  return segmented_sum(ones, segment_ids, num_segments)


def _check_get_norm(arguments: Dict[str, Any], default: Any) -> Any:
  if "norm" in arguments:
    try:
      norm = float(arguments["norm"])
    except (ValueError, TypeError):
      raise ValueError(f"Invalid 'norm' value: {arguments['norm']}. Must be a positive number.")
    if norm <= 0:
      raise ValueError(f"Invalid 'norm' value: {norm}. Must be a positive number.")
    return norm
  return default


_MODES = ("'token-mean', 'sequence-mean-token-mean', 'sequence-mean-token-scale', 'seq-mean-token-sum', "
          "'sequence-mean-token-sum-norm'")


def _f32(x, ref: torch.Tensor) -> torch.Tensor:
  return torch.as_tensor(x, dtype=torch.float32, device=ref.device)


def aggregate_loss(per_token_loss: torch.Tensor, completion_mask: torch.Tensor, loss_agg_mode: str,
                   segment_ids: Optional[torch.Tensor] = None, num_segments: Optional[int] = None,
                   **kwargs: Any) -> WeightedMetric:
  """Aggregates a `[B, T]` per-token loss into a deferred-division `WeightedMetric`.

  Modes: token-mean; sequence-mean-token-mean; sequence-mean-token-scale (norm defaults to the
  row width); seq-mean-token-sum; sequence-mean-token-sum-norm (norm defaults to the batch size).
  With `segment_ids` (packed rows) per-sequence reductions run per segment; segment 0 is padding."""
  ptl = per_token_loss.float()
  m = completion_mask.to(ptl.dtype)
  if segment_ids is not None:
    return _aggregate_loss_segmented(ptl, m, loss_agg_mode, segment_ids, num_segments, **kwargs)
  if loss_agg_mode == "token-mean":
    s, d, md = (ptl * m).sum(), m.sum(), 1.0
  elif loss_agg_mode == "sequence-mean-token-mean":
    cnt = m.sum(-1)
    s = ((ptl * m).sum(-1) / cnt.clamp(min=1.0)).sum()
    d, md = (cnt > 0).sum(), 1.0
  elif loss_agg_mode == "sequence-mean-token-scale":
    norm = _check_get_norm(kwargs, ptl.shape[-1])
    s = ((ptl * m).sum(-1) / max(norm, 1e-6)).sum()
    d, md = (m.sum(-1) > 0).sum(), 1.0
  elif loss_agg_mode == "seq-mean-token-sum":
    act = (m.sum(-1) > 0).float()
    s, d, md = ((ptl * m).sum(-1) * act).sum(), act.sum(), 1e-6
  elif loss_agg_mode == "sequence-mean-token-sum-norm":
    norm = _check_get_norm(kwargs, ptl.shape[0])
    s, d, md = (ptl * m).sum(), norm, 1e-6
  else:
    raise ValueError(f"Unsupported loss aggregation mode: {loss_agg_mode}. Supported modes: {_MODES}.")
  return WeightedMetric(s.float(), _f32(d, ptl), min_denom=md)


def _seg_stats(ptl, m, segment_ids, num_segments):
  if num_segments is None:
    raise ValueError("num_segments must be provided when segment_ids is not None.")
  masked = ptl * m
  l_seg = segmented_sum(masked, segment_ids, num_segments)
  c_seg = segmented_count(segment_ids, num_segments, mask=m)
  a_seg = (c_seg > 0).float()
  a_seg[:, 0] = 0.0
  return masked, l_seg, c_seg, a_seg, a_seg.sum()


def _aggregate_loss_segmented(ptl, m, mode, segment_ids, num_segments, **kwargs) -> WeightedMetric:
  masked, l_seg, c_seg, a_seg, n_act = _seg_stats(ptl, m, segment_ids, num_segments)
  if mode == "token-mean":
    s, d, md = masked.sum(), m.sum(), 1.0
  elif mode == "sequence-mean-token-mean":
    s, d, md = ((l_seg / c_seg.clamp(min=1.0)) * a_seg).sum(), n_act, 1.0
  elif mode == "sequence-mean-token-scale":
    if "norm" not in kwargs:
      raise ValueError("sequence-mean-token-scale under sequence packing requires an explicit 'norm' (e.g. "
                       "max_response_length); the default row-width norm is the pack budget, which dilutes every "
                       "sequence.")
    norm = _check_get_norm(kwargs, ptl.shape[-1])
    s, d, md = ((l_seg / max(norm, 1e-6)) * a_seg).sum(), n_act, 1.0
  elif mode == "seq-mean-token-sum":
    s, d, md = (l_seg * a_seg).sum(), n_act, 1e-6
  elif mode == "sequence-mean-token-sum-norm":
    norm = _check_get_norm(kwargs, n_act)
    s, d, md = masked.sum(), norm, 1e-6
  else:
    raise ValueError(f"Unsupported loss aggregation mode: {mode}. Supported modes: {_MODES}.")
  return WeightedMetric(s.float(), _f32(d, ptl), min_denom=md)


def reduced_loss_agg(per_token_loss: torch.Tensor, completion_mask: torch.Tensor, loss_agg_mode: str,
                     segment_ids: Optional[torch.Tensor] = None, num_segments: Optional[int] = None,
                     **kwargs: Any) -> torch.Tensor:
  """Eager (divide-now) form of `aggregate_loss`, written independently so the two cross-check;
  used only for the `reduced_pg_loss` logging metric. Per-sequence means divide by the number of rows that hold
  at least one unmasked token, exactly like `aggregate_loss` (the reference's eager form averages over all rows,
  tunix/rl/common.py:1003-1014, and so disagrees with its own deferred form on batches with padding rows)."""
  ptl = per_token_loss.float()
  m = completion_mask.to(ptl.dtype)
  if segment_ids is not None:
    masked, l_seg, c_seg, a_seg, n_act = _seg_stats(ptl, m, segment_ids, num_segments)
    if loss_agg_mode == "token-mean":
      return masked.sum() / m.sum().clamp(min=1.0)
    if loss_agg_mode == "sequence-mean-token-mean":
      return ((l_seg / c_seg.clamp(min=1.0)) * a_seg).sum() / n_act.clamp(min=1.0)
    if loss_agg_mode == "sequence-mean-token-scale":
      if "norm" not in kwargs:
        raise ValueError("sequence-mean-token-scale under sequence packing requires an explicit 'norm'")
      norm = _check_get_norm(kwargs, ptl.shape[-1])
      return ((l_seg / max(norm, 1e-6)) * a_seg).sum() / n_act.clamp(min=1.0)
    if loss_agg_mode == "seq-mean-token-sum":
      return (l_seg * a_seg).sum() / n_act.clamp(min=1e-6)
    if loss_agg_mode == "sequence-mean-token-sum-norm":
      norm = _check_get_norm(kwargs, n_act)
      return masked.sum() / _f32(norm, ptl).clamp(min=1e-6)
    raise ValueError(f"Unsupported loss aggregation mode: {loss_agg_mode}. Supported modes: {_MODES}.")
  if loss_agg_mode == "token-mean":
    return (ptl * m).sum() / m.sum().clamp(min=1.0)
  rows = (m.sum(-1) > 0).sum().clamp(min=1)      # rows without a single unmasked token are padding, not sequences
  if loss_agg_mode == "sequence-mean-token-mean":
    return ((ptl * m).sum(-1) / m.sum(-1).clamp(min=1.0)).sum() / rows
  if loss_agg_mode == "sequence-mean-token-scale":
    norm = _check_get_norm(kwargs, ptl.shape[-1])
    return ((ptl * m).sum(-1) / max(norm, 1e-6)).sum() / rows
  if loss_agg_mode == "seq-mean-token-sum":
    act = (m.sum(-1) > 0).float()
    return ((ptl * m).sum(-1) * act).sum() / act.sum().clamp(min=1e-6)
  if loss_agg_mode == "sequence-mean-token-sum-norm":
    norm = _check_get_norm(kwargs, ptl.shape[0])
    return (ptl * m).sum() / max(norm, 1e-6)
  raise ValueError(f"Unsupported loss aggregation mode: {loss_agg_mode}. Supported modes: {_MODES}.")


def _metric_scalar(value: Any) -> Any:
  return value.compute() if isinstance(value, WeightedMetric) else value


def _np(v) -> np.ndarray:
  if isinstance(v, torch.Tensor):
    return v.detach().float().cpu().numpy()
  return np.asarray(v)


def mean_of_means(values: Iterable[Any]) -> np.ndarray:
  """Reducer: mean of per-micro-batch values (WeightedMetrics are divided first)."""
  return np.mean([_np(_metric_scalar(v)) for v in values])


def global_weighted_mean(values: Iterable[WeightedMetric]) -> float:
  """Reducer: sum of numerators over sum of denominators."""
  values = list(values)
  total = sum(float(_np(v.unreduced_sum)) for v in values)
  denom = sum(float(_np(v.denominator)) for v in values)
  return total / denom if denom != 0 else 0.0
