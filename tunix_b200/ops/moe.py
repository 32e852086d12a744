"""Grouped expert MLP: rows sorted by expert, one GEMM chain per expert over its row range.

`grouped_mlp(xs, counts, gate_up [E,2F,D], down [E,D,F])` is the single-rank form of the
reference's three grouped matmuls (tunix/models/qwen3/model.py:975-995)."""
from __future__ import annotations

from typing import List

import torch

from . import functional as F


def grouped_mlp(xs: torch.Tensor, counts: List[int], gate_up: torch.Tensor, down: torch.Tensor, kind: str,
                first_expert: int = 0) -> torch.Tensor:
  outs = []
  start = 0
  for e, c in enumerate(counts):
    if c == 0:
      continue
    x = xs[start:start + c]
    h = F.glu(F.linear(x, gate_up[first_expert + e]), kind)
    outs.append(F.linear(h, down[first_expert + e]))
    start += c
  if not outs:
    return xs.new_zeros(xs.shape)
  return torch.cat(outs, dim=0)
