"""Flash attention on the sm_100a kernels.

Forward: `tx_flash_fwd` (tcgen05 / TMEM, head_dim 128, causal or full, GQA, strided q/k/v views
of a fused projection). Backward: `tx_flash_bwd`, two tcgen05 kernels (dK/dV per key tile, dQ per
query tile) with a fixed reduction order, so gradients are bitwise reproducible.
"""
from __future__ import annotations

import os
from typing import Any, Tuple

import torch

from . import _lib

_DISABLED = os.environ.get("TUNIX_B200_FLASH", "1") == "0"


def _rows_ok(t: torch.Tensor) -> bool:
  # [B, L, heads, H] view whose (B, L) flatten to rows of one stride and heads*H is contiguous
  B, L, n, H = t.shape
  sb, sl, sn, sh = t.stride()
  return sh == 1 and sn == H and (B == 1 or sb == L * sl) and sl % 8 == 0 and t.data_ptr() % 16 == 0


def supported(q, k, v, mask, causal) -> bool:
  if _DISABLED or mask is not None or not q.is_cuda or q.dtype != torch.bfloat16:
    return False
  if q.dim() != 4 or q.shape[-1] != 128 or k.shape[-1] != 128 or q.shape[2] % k.shape[2] != 0:
    return False
  if k.shape != v.shape or k.dtype != q.dtype or v.dtype != q.dtype:
    return False
  return _rows_ok(q) and _rows_ok(k) and _rows_ok(v) and _lib.available()


def segment_bounds(segment_ids: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
  """[B, L] segment ids of packed rows (equal ids are contiguous) -> int32 (first, last) token index
  of every token's segment. Padding (id 0) forms segments of its own and only ever sees itself."""
  B, L = segment_ids.shape
  idx = torch.arange(L, device=segment_ids.device, dtype=torch.int32).expand(B, L)
  change = torch.ones((B, L), dtype=torch.bool, device=segment_ids.device)
  change[:, 1:] = segment_ids[:, 1:] != segment_ids[:, :-1]
  lo = torch.cummax(torch.where(change, idx, torch.zeros_like(idx)), dim=1).values
  last = torch.ones((B, L), dtype=torch.bool, device=segment_ids.device)
  last[:, :-1] = change[:, 1:]
  big = torch.full_like(idx, L - 1)
  hi = torch.flip(torch.cummin(torch.flip(torch.where(last, idx, big), [1]), dim=1).values, [1])
  return lo.to(torch.int32).contiguous(), hi.to(torch.int32).contiguous()


def forward(q, k, v, *, causal: bool, scale: float, segments=None) -> Tuple[torch.Tensor, Any]:
  """q [B,Lq,N,128], k/v [B,Lk,K,128] -> (o [B,Lq,N,128] contiguous, ctx). `segments` is the
  (first, last) pair of `segment_bounds` for packed rows (needs Lq == Lk)."""
  B, Lq, N, H = q.shape
  Lk, Kh = k.shape[1], k.shape[2]
  o = torch.empty((B, Lq, N, H), dtype=q.dtype, device=q.device)
  lse = torch.empty((B, N, Lq), dtype=torch.float32, device=q.device)
  lib = _lib.require()
  lo, hi = segments if segments is not None else (None, None)
  rc = lib.tx_flash_fwd_seg(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(), B, N, Kh, Lq,
                            Lk, H, q.stride(1), k.stride(1), v.stride(1), N * H, int(causal), float(scale),
                            lo.data_ptr() if lo is not None else None, hi.data_ptr() if hi is not None else None,
                            _lib.status_word(q.device).data_ptr(), _lib.stream_ptr())
  _lib.check_rc(rc, "tx_flash_fwd_seg")
  return o, ("tx", lse, causal, scale, segments)


_BWD_LIBRARY = os.environ.get("TUNIX_B200_FLASH_BWD", "1") == "0"


def backward(do, q, k, v, o, ctx, dq_out, dk_out, dv_out) -> None:
  """Writes dq/dk/dv ([B,L,heads,128], may be strided views of one fused gradient buffer)."""
  _, lse, causal, scale = ctx[:4]
  segments = ctx[4] if len(ctx) > 4 else None
  B, Lq, N, H = q.shape
  Lk, Kh = k.shape[1], k.shape[2]
  if _BWD_LIBRARY and segments is None:
    e = torch.empty(0, dtype=torch.long, device=q.device)
    dq, dk, dv = torch.ops.aten._scaled_dot_product_flash_attention_backward(
        do.transpose(1, 2), q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), o.transpose(1, 2), lse,
        None, None, Lq, Lk, 0.0, causal, e, e, scale=scale)
    dq_out.copy_(dq.transpose(1, 2))
    dk_out.copy_(dk.transpose(1, 2))
    dv_out.copy_(dv.transpose(1, 2))
    return
  if not _rows_ok(do):
    do = do.contiguous()
  outs = [t if _rows_ok(t) else torch.empty(t.shape, dtype=t.dtype, device=t.device) for t in (dq_out, dk_out, dv_out)]
  delta = torch.empty((B, N, Lq), dtype=torch.float32, device=q.device)
  lib = _lib.require()
  lo, hi = segments if segments is not None else (None, None)
  rc = lib.tx_flash_bwd_seg(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), do.data_ptr(), lse.data_ptr(),
                            delta.data_ptr(), outs[0].data_ptr(), outs[1].data_ptr(), outs[2].data_ptr(), B, N, Kh,
                            Lq, Lk, H, q.stride(1), k.stride(1), v.stride(1), o.stride(1), do.stride(1),
                            outs[0].stride(1), outs[1].stride(1), outs[2].stride(1), int(causal), float(scale),
                            lo.data_ptr() if lo is not None else None, hi.data_ptr() if hi is not None else None,
                            _lib.status_word(q.device).data_ptr(), _lib.stream_ptr())
  _lib.check_rc(rc, "tx_flash_bwd_seg")
  for dst, src in zip((dq_out, dk_out, dv_out), outs):
    if dst is not src:
      dst.copy_(src)


class _FlashFn(torch.autograd.Function):
  @staticmethod
  def forward(ctx, q, k, v, causal, scale, seg_lo=None, seg_hi=None):
    segments = (seg_lo, seg_hi) if seg_lo is not None else None
    o, c = forward(q, k, v, causal=causal, scale=scale, segments=segments)
    ctx.save_for_backward(q, k, v, o, c[1])
    ctx.causal, ctx.scale, ctx.segments = causal, scale, segments
    return o

  @staticmethod
  def backward(ctx, do):
    q, k, v, o, lse = ctx.saved_tensors
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    backward(do.contiguous(), q, k, v, o, ("tx", lse, ctx.causal, ctx.scale, ctx.segments), dq, dk, dv)
    return dq, dk, dv, None, None, None, None


class _FlashPackedFn(torch.autograd.Function):
  """Attention over one packed [B, L, N + 2K, 128] tensor (the layout the fused q|k|v projection produces). The
  backward writes dq, dk and dv straight into the slices of ONE gradient buffer, which spares autograd the three
  zero-filled full-size tensors, three slice copies and two adds it needs for separate q/k/v gradients."""

  @staticmethod
  def forward(ctx, qkv, N, K, causal, scale, seg_lo=None, seg_hi=None):
    segments = (seg_lo, seg_hi) if seg_lo is not None else None
    q, k, v = qkv[:, :, :N], qkv[:, :, N:N + K], qkv[:, :, N + K:]
    o, c = forward(q, k, v, causal=causal, scale=scale, segments=segments)
    ctx.save_for_backward(qkv, o, c[1])
    ctx.cfg = (N, K, causal, scale, segments)
    return o

  @staticmethod
  def backward(ctx, do):
    qkv, o, lse = ctx.saved_tensors
    N, K, causal, scale, segments = ctx.cfg
    dqkv = torch.empty(qkv.shape, dtype=qkv.dtype, device=qkv.device)
    backward(do.contiguous(), qkv[:, :, :N], qkv[:, :, N:N + K], qkv[:, :, N + K:], o,
             ("tx", lse, causal, scale, segments), dqkv[:, :, :N], dqkv[:, :, N:N + K], dqkv[:, :, N + K:])
    return dqkv, None, None, None, None, None, None


def packed_supported(qkv: torch.Tensor, N: int, K: int) -> bool:
  return (qkv.dim() == 4 and qkv.is_contiguous() and qkv.shape[2] == N + 2 * K and
          supported(qkv[:, :, :N], qkv[:, :, N:N + K], qkv[:, :, N + K:], None, True))


def flash_attention_packed(qkv, N: int, K: int, *, causal: bool, scale: float, segments=None):
  lo, hi = segments if segments is not None else (None, None)
  return _FlashPackedFn.apply(qkv, N, K, causal, scale, lo, hi)


def flash_attention(q, k, v, *, causal: bool, scale: float, segment_ids=None):
  """`segment_ids` [B, L]: tokens attend only within their own (contiguous) segment."""
  if segment_ids is not None:
    lo, hi = segment_bounds(segment_ids)
    return _FlashFn.apply(q, k, v, causal, scale, lo, hi)
  return _FlashFn.apply(q, k, v, causal, scale)
