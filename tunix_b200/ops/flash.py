"""Flash attention on the sm_100a kernels (forward and backward)."""
from __future__ import annotations

import torch


def supported(q, k, v, mask, causal) -> bool:
  return False


def forward(q, k, v, *, causal: bool, scale: float):
  raise NotImplementedError


def backward(do, q, k, v, o, ctx, dq_out, dk_out, dv_out):
  raise NotImplementedError


def flash_attention(q, k, v, *, causal: bool, scale: float):
  raise NotImplementedError
