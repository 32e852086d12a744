"""The batch contract of diffusion objectives (tunix/diffusion/types.py).

A `DiffusionTokenBatch` is target-aligned: `target_ids` [batch, length] integers,
`loss_weights` of the same shape (real or boolean, finite, non-negative; active targets are
non-negative ids), and `model_inputs`, any nesting of dicts / lists / tuples of batch-major
tensors or NumPy arrays that a model-specific scorer consumes.
"""
from __future__ import annotations

import dataclasses
from typing import Any, Iterator, Tuple

import numpy as np
import torch

Array = Any          # torch.Tensor | np.ndarray
ModelInputs = Any    # nesting of Array


def _leaves(tree: Any) -> Iterator[Any]:
  if isinstance(tree, dict):
    for k in sorted(tree):
      yield from _leaves(tree[k])
  elif isinstance(tree, (list, tuple)):
    for v in tree:
      yield from _leaves(v)
  elif tree is not None:
    yield tree


def _shape_and_kind(name: str, v: Any) -> Tuple[Tuple[int, ...], str]:
  """kind is one of 'bool', 'int', 'float', 'other'."""
  if isinstance(v, torch.Tensor):
    if v.dtype == torch.bool:
      kind = "bool"
    elif v.dtype.is_floating_point:
      kind = "float"
    elif v.dtype.is_complex:
      kind = "other"
    else:
      kind = "int"
    return tuple(v.shape), kind
  if isinstance(v, np.ndarray):
    kind = {"b": "bool", "i": "int", "u": "int", "f": "float"}.get(v.dtype.kind, "other")
    return tuple(v.shape), kind
  raise TypeError(f"{name} must be a torch.Tensor or a NumPy array, got {type(v).__name__}")


def _host(v: Any) -> np.ndarray:
  return v.detach().float().cpu().numpy() if isinstance(v, torch.Tensor) else np.asarray(v)


@dataclasses.dataclass(frozen=True)
class DiffusionTokenBatch:
  model_inputs: ModelInputs
  target_ids: Array
  loss_weights: Array

  @classmethod
  def create(cls, *, model_inputs: ModelInputs, target_ids: Array, loss_weights: Array) -> "DiffusionTokenBatch":
    return cls(model_inputs=model_inputs, target_ids=target_ids, loss_weights=loss_weights).validate()

  def validate(self, check_values: bool = True) -> "DiffusionTokenBatch":
    """Shape/dtype checks always; value checks (a device-to-host read) unless `check_values=False`."""
    tshape, tkind = _shape_and_kind("target_ids", self.target_ids)
    if len(tshape) != 2:
      raise ValueError(f"target_ids must have shape [batch, length]; received {tshape}")
    if tkind != "int":
      raise TypeError("target_ids must have an integer dtype")
    wshape, wkind = _shape_and_kind("loss_weights", self.loss_weights)
    if wshape != tshape:
      raise ValueError(f"loss_weights must match target_ids shape; received {wshape} and {tshape}")
    if wkind == "other":
      raise TypeError("loss_weights must have a real numeric or boolean dtype")
    if check_values:
      w = _host(self.loss_weights)
      if not np.all(np.isfinite(w)):
        raise ValueError("loss_weights must contain only finite values")
      if np.any(w < 0):
        raise ValueError("loss_weights must be nonnegative")
      t = _host(self.target_ids)
      if np.any(t[w > 0] < 0):
        raise ValueError("active target_ids must be nonnegative")
    leaves = list(_leaves(self.model_inputs))
    if not leaves:
      raise ValueError("model_inputs must contain at least one array")
    for i, leaf in enumerate(leaves):
      shape, kind = _shape_and_kind(f"model_inputs leaf {i}", leaf)
      if not shape:
        raise ValueError(f"model_inputs leaf {i} must be batch-major, not scalar")
      if shape[0] != tshape[0]:
        raise ValueError(f"model_inputs leaf {i} has batch size {shape[0]}; expected {tshape[0]}")
      if kind == "other":
        raise TypeError(f"model_inputs leaf {i} must have a real numeric or boolean dtype")
    return self


def validate_diffusion_logits(batch: DiffusionTokenBatch, logits: Array) -> Array:
  """Logits must be floating point [batch, length, vocabulary] aligned with the batch's targets."""
  shape, kind = _shape_and_kind("logits", logits)
  tshape = tuple(batch.target_ids.shape)
  if len(shape) != 3:
    raise ValueError(f"diffusion logits must have shape [batch, length, vocabulary]; received {shape}")
  if shape[:2] != tshape:
    raise ValueError(f"diffusion logits must align with target_ids; received {shape[:2]} and {tshape}")
  if shape[2] <= 0:
    raise ValueError("diffusion logits must have a non-empty vocabulary axis")
  if kind != "float":
    raise TypeError("diffusion logits must have a floating-point dtype")
  return logits
