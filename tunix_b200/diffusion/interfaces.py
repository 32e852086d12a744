"""Callable contracts that plug a diffusion model into the trainers (tunix/diffusion/interfaces.py)."""
from __future__ import annotations

from typing import Protocol, TypeVar

import torch

from . import types

RawBatchT_contra = TypeVar("RawBatchT_contra", contravariant=True)


class DiffusionBatchAdapter(Protocol[RawBatchT_contra]):
  """Turns a data-pipeline batch into the canonical target-aligned batch."""

  def __call__(self, batch: RawBatchT_contra, /) -> types.DiffusionTokenBatch:
    ...


class DiffusionLogitsFn(Protocol):
  """Scores a prepared batch: returns [batch, length, vocabulary] logits aligned with the targets."""

  def __call__(self, model: torch.nn.Module, model_inputs: types.ModelInputs, /) -> types.Array:
    ...


def compute_diffusion_logits(model: torch.nn.Module, batch: types.DiffusionTokenBatch,
                             logits_fn: DiffusionLogitsFn, check_values: bool = False) -> types.Array:
  batch.validate(check_values=check_values)
  return types.validate_diffusion_logits(batch, logits_fn(model, batch.model_inputs))


def masked_token_loss(model: torch.nn.Module, batch: types.DiffusionTokenBatch, logits_fn: DiffusionLogitsFn):
  """Weighted token cross-entropy of a diffusion batch as (sum of weighted losses, sum of weights):
  the unreduced pair the trainers accumulate across micro-batches."""
  logits = compute_diffusion_logits(model, batch, logits_fn)
  w = torch.as_tensor(batch.loss_weights, device=logits.device).float()
  t = torch.as_tensor(batch.target_ids, device=logits.device).long().clamp_min(0)
  logp = torch.log_softmax(logits.float(), dim=-1).gather(-1, t[..., None]).squeeze(-1)
  return -(logp * w).sum(), w.sum()
