"""CUDA attention entry points.

Layout convention: q [B,T,N,H], k/v [B,S,K,H] (token-major, heads contiguous) - what the fused
qkv projection produces, so q, k and v may be strided views of one buffer and no transposes are
materialised on the way in.

`flash_fwd` / `flash_bwd` are the explicit forward / backward pair used by hand-scheduled
backward passes; `attention_cuda` is the autograd-facing call. The sm_100a kernels in `flash.py`
are used when they cover the case, otherwise the library flash kernels behind
`torch.ops.aten._scaled_dot_product_flash_attention`.
"""
from __future__ import annotations

from typing import Any, Optional, Tuple

import torch
import torch.nn.functional as F

from . import flash


class SegmentMask:
  """Causal attention restricted to contiguous segments of packed rows, kept symbolic.

  It travels where a dense [B, T, S] mask would; the sm_100a kernels consume the (first, last)
  bounds directly, every other path asks for `dense()` (built once). Query rows of padding
  (segment id 0) see nothing in the dense form and only themselves in the kernels; both are
  excluded from losses."""

  def __init__(self, segment_ids: torch.Tensor):
    self.segment_ids = segment_ids
    self._dense = None
    self._bounds = None

  def bounds(self):
    if self._bounds is None:
      self._bounds = flash.segment_bounds(self.segment_ids)
    return self._bounds

  def dense(self) -> torch.Tensor:
    if self._dense is None:
      seg = self.segment_ids
      L = seg.shape[1]
      tri = torch.ones(L, L, dtype=torch.bool, device=seg.device).tril()[None]
      self._dense = (seg[:, :, None] == seg[:, None, :]) & tri & (seg[:, :, None] != 0)
    return self._dense


def flash_fwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, causal: bool, scale: float,
              segments=None) -> Tuple[torch.Tensor, Any]:
  """Returns (o [B,T,N,H] contiguous, ctx for `flash_bwd`). `segments`: bounds of a `SegmentMask`
  (only with the sm_100a kernel; callers check `flash.supported` first)."""
  if flash.supported(q, k, v, None, causal):
    return flash.forward(q, k, v, causal=causal, scale=scale, segments=segments)
  if segments is not None:
    raise ValueError("packed segments need the sm_100a flash kernel (bf16, head_dim 128)")
  qt, kt, vt = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
  rep = qt.shape[1] // kt.shape[1]
  try:
    res = torch.ops.aten._scaled_dot_product_flash_attention(qt, kt, vt, 0.0, causal, False, scale=scale)
  except RuntimeError:
    if rep == 1:
      raise
    kt, vt = kt.repeat_interleave(rep, dim=1), vt.repeat_interleave(rep, dim=1)
    res = torch.ops.aten._scaled_dot_product_flash_attention(qt, kt, vt, 0.0, causal, False, scale=scale)
    o, lse, cq, ck, mq, mk, seed, offset, _ = res
    return o.transpose(1, 2).contiguous(), ("aten_rep", lse, cq, ck, mq, mk, seed, offset, causal, scale, rep)
  o, lse, cq, ck, mq, mk, seed, offset, _ = res
  return o.transpose(1, 2).contiguous(), ("aten", lse, cq, ck, mq, mk, seed, offset, causal, scale, 1)


def flash_bwd(do: torch.Tensor, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, o: torch.Tensor, ctx: Any,
              dq_out: torch.Tensor, dk_out: torch.Tensor, dv_out: torch.Tensor) -> None:
  """Writes dq/dk/dv (token-major [B,T,heads,H], may be strided views) given do and the forward ctx."""
  if ctx[0] == "tx":
    flash.backward(do, q, k, v, o, ctx, dq_out, dk_out, dv_out)
    return
  kind, lse, cq, ck, mq, mk, seed, offset, causal, scale, rep = ctx
  qt, kt, vt = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
  if kind == "aten_rep":
    kt, vt = kt.repeat_interleave(rep, dim=1), vt.repeat_interleave(rep, dim=1)
  dq, dk, dv = torch.ops.aten._scaled_dot_product_flash_attention_backward(
      do.transpose(1, 2), qt, kt, vt, o.transpose(1, 2), lse, cq, ck, mq, mk, 0.0, causal, seed, offset, scale=scale)
  if kind == "aten_rep":
    B, NK, S, H = dk.shape
    dk = dk.view(B, NK // rep, rep, S, H).sum(2)
    dv = dv.view(B, NK // rep, rep, S, H).sum(2)
  dq_out.copy_(dq.transpose(1, 2))
  dk_out.copy_(dk.transpose(1, 2))
  dv_out.copy_(dv.transpose(1, 2))


def attention_cuda(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, mask: Optional[torch.Tensor],
                   causal: bool, scale: float) -> torch.Tensor:
  if isinstance(mask, SegmentMask):
    if q.shape[1] == k.shape[1] and flash.supported(q, k, v, None, True):
      lo, hi = mask.bounds()
      return flash._FlashFn.apply(q, k, v, True, scale, lo, hi)
    mask = mask.dense()
  if flash.supported(q, k, v, mask, causal):
    return flash.flash_attention(q, k, v, causal=causal, scale=scale)
  qt, kt, vt = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
  attn_mask = None
  is_causal = causal and mask is None
  if is_causal and q.shape[1] != k.shape[1]:
    # the library's causal flag aligns the triangle to the first key; here queries are the LAST rows of the keys
    T, S = q.shape[1], k.shape[1]
    mask = torch.ones(T, S, dtype=torch.bool, device=q.device).tril(S - T)[None]
    is_causal = False
  if mask is not None:
    attn_mask = mask[:, None, :, :]
  o = F.scaled_dot_product_attention(qt, kt, vt, attn_mask=attn_mask, is_causal=is_causal, scale=scale,
                                     enable_gqa=qt.shape[1] != kt.shape[1])
  return o.transpose(1, 2)
