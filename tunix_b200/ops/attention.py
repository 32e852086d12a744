"""CUDA attention entry point used by `functional.attention`.

Layout convention: q [B,T,N,H], k/v [B,S,K,H] (token-major, heads contiguous), which is what
the fused qkv projection produces, so no transposes are materialised on the way in.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn.functional as F


def attention_cuda(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, mask: Optional[torch.Tensor],
                   causal: bool, scale: float) -> torch.Tensor:
  """Dispatches to the flash kernels in this package when they cover the case, otherwise to
  the library kernel behind `scaled_dot_product_attention`."""
  from . import flash
  if flash.supported(q, k, v, mask, causal):
    return flash.flash_attention(q, k, v, causal=causal, scale=scale)
  qt, kt, vt = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
  attn_mask = None
  is_causal = causal and mask is None
  if mask is not None:
    attn_mask = mask[:, None, :, :]
  o = F.scaled_dot_product_attention(qt, kt, vt, attn_mask=attn_mask, is_causal=is_causal, scale=scale,
                                     enable_gqa=qt.shape[1] != kt.shape[1])
  return o.transpose(1, 2)
