"""Flash attention on the sm_100a kernels (forward and backward)."""
from __future__ import annotations

import torch


def supported(q, k, v, mask, causal) -> bool:
  return False


def flash_attention(q, k, v, *, causal: bool, scale: float):
  raise NotImplementedError
