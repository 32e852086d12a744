"""Average pooling of an N-d array down to a target shape (every axis is pooled).

Same window/stride rule as tunix/distillation/feature_extraction/pooling.py:33-131:
VALID: stride = in // out, window = in - (out-1)*stride; SAME: stride = window = ceil(in/out)
with zero padding split low/high and the divisor either the window size or the count of real
elements. Implemented as one cumulative-sum box filter per pooled axis, so any rank works.
"""
from __future__ import annotations

import enum
from typing import Sequence

import torch


class PaddingMode(enum.Enum):
  VALID = "VALID"
  SAME = "SAME"


def _pool_axis(x: torch.Tensor, axis: int, out: int, mode: PaddingMode, include_pad: bool) -> torch.Tensor:
  n = x.shape[axis]
  if out == n:
    return x
  if mode == PaddingMode.VALID:
    stride = n // out
    window = n - (out - 1) * stride
    lo = 0
  else:
    stride = window = (n + out - 1) // out
    total = max((out - 1) * stride + window - n, 0)
    lo = total // 2
  x = x.movedim(axis, -1)
  starts = torch.arange(out, device=x.device) * stride - lo
  ends = starts + window
  s_c, e_c = starts.clamp(0, n), ends.clamp(0, n)
  cs = torch.nn.functional.pad(torch.cumsum(x.to(torch.float64 if x.dtype == torch.float64 else torch.float32), -1),
                               (1, 0))
  sums = cs.index_select(-1, e_c) - cs.index_select(-1, s_c)
  if mode == PaddingMode.SAME and not include_pad:
    div = (e_c - s_c).to(sums.dtype)
  else:
    div = torch.full_like(e_c, window).to(sums.dtype)
  if sums.shape[-1] != out:
    raise ValueError(f"pooling produced {sums.shape[-1]} elements, wanted {out}")
  return (sums / div).to(x.dtype).movedim(-1, axis)


def avg_pool_array_to_target_shape(input_array: torch.Tensor, target_shape: Sequence[int],
                                   padding_mode: PaddingMode = PaddingMode.VALID,
                                   count_include_pad_for_same_padding: bool = False) -> torch.Tensor:
  target_shape = tuple(int(t) for t in target_shape)
  if tuple(input_array.shape) == target_shape:
    return input_array
  if input_array.ndim != len(target_shape):
    raise ValueError(f"Input array rank ({input_array.ndim}) must match target_shape rank ({len(target_shape)}).")
  for i, (t, n) in enumerate(zip(target_shape, input_array.shape)):
    if not 1 <= t <= n:
      raise ValueError(f"Target dimension target_shape[{i}]={t} is invalid. Must be 1 <= target_dim <= input_dim ({n}).")
  out = input_array
  for ax, t in enumerate(target_shape):
    out = _pool_axis(out, ax, t, padding_mode, count_include_pad_for_same_padding)
  if tuple(out.shape) != target_shape:
    raise ValueError(f"pooled shape {tuple(out.shape)} does not match target_shape {target_shape}")
  return out
