"""Vocabulary-parallel lm_head + selective log-softmax (+ entropy): every rank of a tensor-parallel
group holds rows [v0, v0 + V/tp) of the head, and neither the [T, V] logits nor a [T, V/tp] slice
of them is ever resident beyond one sequence chunk.

Per chunk each rank runs the same two kernels as the single-rank path (`kernels.gemm` into an fp32
block, `kernels.logprob_fwd` over it) on its slice, with the targets shifted by v0: a target owned
by another rank is out of range for the kernel, which then reports 0 for it. What crosses the ranks
is three numbers per token - the local log-sum-exp, the local target logit and the local entropy -
in ONE all-gather; they combine exactly:

  lse   = log sum_r exp(lse_r)                    target logit = sum_r zt_r
  H     = lse - sum_r exp(lse_r - lse) (lse_r - H_r)          logp = target logit - lse

The backward kernel takes the log-sum-exp as an input, so handing it the GLOBAL one yields the
global softmax directly; the one-hot term only fires on the owning rank. dW stays local, dh is a
partial sum and is all-reduced. Reference: the chunked scan of tunix/rl/common.py:485-571 (which
relies on XLA to partition the vocabulary axis).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.distributed as dist

bf16 = torch.bfloat16


def _use_kernels(h: torch.Tensor, w: torch.Tensor) -> bool:
  return h.is_cuda and h.dtype == bf16 and w.dtype == bf16 and w.shape[0] % 8 == 0 and w.shape[1] % 8 == 0


def _local_forward(h, w, tgt, inv_temp, softcap, want_entropy, buf):
  """(target logit or 0, local lse, local entropy or None) of one chunk on this rank's vocabulary slice."""
  V = w.shape[0]
  if buf is not None:
    from . import kernels
    lg = kernels.gemm(h, w, out=buf[:h.shape[0]])
    lp, lse, ent = kernels.logprob_fwd(lg, tgt, inv_temp, softcap, want_entropy)
    own = (tgt >= 0) & (tgt < V)
    return torch.where(own, lp + lse, torch.zeros_like(lp)), lse, ent
  z = h.float() @ w.float().t()
  if softcap > 0:
    z = softcap * torch.tanh(z / softcap)
  z = z * inv_temp
  lse = torch.logsumexp(z, -1)
  own = (tgt >= 0) & (tgt < V)
  zt = torch.where(own, z.gather(1, tgt.clamp(0, V - 1).long()[:, None])[:, 0], torch.zeros_like(lse))
  ent = None
  if want_entropy:
    p = torch.exp(z - lse[:, None])
    ent = lse - (p * z).sum(-1)
  return zt, lse, ent


def _local_dlogits(h, w, tgt, lse, ent, g_logp, g_ent, inv_temp, softcap, buf, dbuf):
  V = w.shape[0]
  if buf is not None:
    from . import kernels
    lg = kernels.gemm(h, w, out=buf[:h.shape[0]])
    return kernels.logprob_bwd(lg, tgt, lse, ent, g_logp, g_ent, inv_temp, softcap, out=dbuf[:h.shape[0]])
  raw = h.float() @ w.float().t()
  z, dcap = raw, 1.0
  if softcap > 0:
    th = torch.tanh(raw / softcap)
    z, dcap = softcap * th, 1.0 - th * th
  z = z * inv_temp
  p = torch.exp(z - lse[:, None])
  onehot = torch.zeros_like(p)
  own = (tgt >= 0) & (tgt < V)
  rows = torch.nonzero(own)[:, 0]
  onehot[rows, tgt[rows].long()] = 1.0
  d = torch.zeros_like(p)
  if g_logp is not None:
    d = d + g_logp[:, None] * (onehot - p)
  if g_ent is not None:
    d = d - g_ent[:, None] * p * (z - lse[:, None] + ent[:, None])
  return (d * inv_temp * dcap).to(h.dtype)


class _VocabParallelLogprob(torch.autograd.Function):

  @staticmethod
  def forward(ctx, h2, w, targets, group, v0, inv_temp, softcap, want_entropy, rows):
    T, D = h2.shape
    V = w.shape[0]
    tp = dist.get_world_size(group)
    fast = _use_kernels(h2, w)
    tgt = (targets.to(torch.int64) - v0).clamp(-1, V).to(torch.int32)      # out of range: another rank's target
    buf = torch.empty((rows, V), dtype=torch.float32, device=h2.device) if fast else None
    stats = torch.zeros((3, T), dtype=torch.float32, device=h2.device)     # zt, lse, entropy of this rank
    for s in range(0, T, rows):
      e = min(T, s + rows)
      zt, lse, ent = _local_forward(h2[s:e], w, tgt[s:e], inv_temp, softcap, want_entropy, buf)
      stats[0, s:e], stats[1, s:e] = zt, lse
      if want_entropy:
        stats[2, s:e] = ent
    every = torch.empty((tp, 3, T), dtype=torch.float32, device=h2.device)
    dist.all_gather_into_tensor(every, stats, group=group) if dist.get_backend(group) != "gloo" else \
        dist.all_gather(list(every.unbind(0)), stats, group=group)
    lse_r = every[:, 1]
    lse = torch.logsumexp(lse_r, 0)
    logp = every[:, 0].sum(0) - lse
    ent = None
    if want_entropy:
      ent = lse - (torch.exp(lse_r - lse[None]) * (lse_r - every[:, 2])).sum(0)
    ctx.save_for_backward(h2, w, tgt, lse, ent)
    ctx.cfg = (group, inv_temp, softcap, rows, fast)
    return logp, ent

  @staticmethod
  def backward(ctx, g_logp, g_ent):
    h2, w, tgt, lse, ent = ctx.saved_tensors
    group, inv_temp, softcap, rows, fast = ctx.cfg
    T, D = h2.shape
    V = w.shape[0]
    need_dh, need_dw = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
    g_logp = g_logp.contiguous().float() if g_logp is not None else None
    g_ent = g_ent.contiguous().float() if (g_ent is not None and ent is not None) else None
    buf = torch.empty((rows, V), dtype=torch.float32, device=h2.device) if fast else None
    dbuf = torch.empty((rows, V), dtype=bf16, device=h2.device) if fast else None
    dh = torch.zeros_like(h2) if need_dh else None
    mg = getattr(w, "main_grad", None) if need_dw else None
    dw_acc = torch.zeros((V, D), dtype=torch.float32, device=h2.device) if (need_dw and mg is None) else None
    for s in range(0, T, rows):
      e = min(T, s + rows)
      dl = _local_dlogits(h2[s:e], w, tgt[s:e], lse[s:e], ent[s:e] if ent is not None else None,
                          g_logp[s:e] if g_logp is not None else None, g_ent[s:e] if g_ent is not None else None,
                          inv_temp, softcap, buf, dbuf)
      if fast:
        from . import kernels
        if need_dh:
          kernels.gemm(dl, w, b_mn=True, out=dh[s:e])
        if need_dw:
          kernels.gemm(dl, h2[s:e], a_mn=True, b_mn=True, out=mg if mg is not None else dw_acc, accumulate=True)
      else:
        if need_dh:
          dh[s:e] = (dl.float() @ w.float()).to(h2.dtype)
        if need_dw:
          (mg if mg is not None else dw_acc).add_(dl.float().t() @ h2[s:e].float())
    if need_dh:
      dist.all_reduce(dh, group=group)             # every rank contributed its vocabulary slice's share
    dw = None if (not need_dw or mg is not None) else dw_acc.to(w.dtype)
    return dh, dw, None, None, None, None, None, None, None


def linear_logprob(hidden: torch.Tensor, weight_shard: torch.Tensor, targets: torch.Tensor, group, vocab_start: int,
                   temperature: float = 1.0, softcap: float = 0.0,
                   want_entropy: bool = False) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
  """hidden [..., D] (replicated over the group), weight_shard [V / tp, D], targets [...] (global ids) ->
  (logp [...], entropy [...] or None), fp32, identical on every rank of the group."""
  from .functional import _chunk_rows
  lead = targets.shape
  D = hidden.shape[-1]
  inv_temp = 1.0 if temperature in (0.0, 1.0) else 1.0 / temperature
  h2 = hidden.reshape(-1, D).contiguous()
  T = h2.shape[0]
  tg = targets.reshape(-1)
  pad = (-T) % 8
  if pad:
    h2 = torch.cat([h2, h2.new_zeros(pad, D)], 0)
    tg = torch.cat([tg, tg.new_zeros(pad)], 0)
  rows = _chunk_rows(h2.shape[0], weight_shard.shape[0])
  lp, ent = _VocabParallelLogprob.apply(h2, weight_shard, tg, group, int(vocab_start), inv_temp, float(softcap),
                                        bool(want_entropy), rows)
  return lp[:T].view(lead), (ent[:T].view(lead) if ent is not None else None)
