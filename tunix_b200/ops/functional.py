"""Differentiable hot ops.

Every function here accepts CPU or CUDA tensors. CUDA bf16 tensors run on the hand-written
sm_100a kernels (`kernels.py`) through `torch.autograd.Function`s with explicit backward
passes; everything else runs the PyTorch statement in `ref.py` under ordinary autograd.

Gradient accumulation fusion: a parameter may carry a `main_grad` attribute (an fp32 tensor
of the same shape). The backward passes then add the weight gradient straight into it from
the GEMM epilogue / reduction kernel and return no `.grad`, so accumulation over
micro-batches costs no extra pass and no bf16 rounding.
"""
from __future__ import annotations

import math
import threading
from typing import Optional, Tuple

import torch
import torch.nn.functional as F

from . import _lib, kernels, ref

bf16 = torch.bfloat16


def _use_kernels(*ts: torch.Tensor) -> bool:
  t = ts[0]
  if not t.is_cuda:
    return False
  if t.dtype != bf16:
    return False
  _lib.require()  # a CUDA bf16 tensor without the library is an error, never a silent fallback
  return True


def _main_grad(p: torch.Tensor) -> Optional[torch.Tensor]:
  return getattr(p, "main_grad", None)


# ------------------------------------------------------------------------------ linear
class _LinearFn(torch.autograd.Function):

  @staticmethod
  def forward(ctx, x2, w, holder):
    ctx.save_for_backward(x2, w)
    ctx.holder = holder
    return kernels.gemm(x2, w)

  @staticmethod
  def backward(ctx, dy):
    x2, w = ctx.saved_tensors
    dy = dy.contiguous()
    dx = dw = None
    if ctx.needs_input_grad[0]:
      dx = kernels.gemm(dy, w, b_mn=True)                      # dx[M,K] = dy[M,N] @ w[N,K]
    if ctx.needs_input_grad[1]:
      mg = _main_grad(ctx.holder) if ctx.holder is not None else None
      if mg is not None:
        kernels.gemm(dy, x2, a_mn=True, b_mn=True, out=mg, accumulate=True)   # dw[N,K] += dy^T @ x
      else:
        dw = kernels.gemm(dy, x2, a_mn=True, b_mn=True)
    return dx, dw, None


def linear(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
  """y = x @ w^T (+ bias); w is [out, in]."""
  if _use_kernels(x, w) and w.dtype == bf16:
    K = x.shape[-1]
    x2 = x.reshape(-1, K)
    if not x2.is_contiguous():
      x2 = x2.contiguous()
    M, N = x2.shape[0], w.shape[0]
    if (M <= 128 and not (torch.is_grad_enabled() and (x.requires_grad or w.requires_grad))
        and kernels.gemm_skinny_supported(x2, w) and (bias is None or (bias.dtype == bf16 and bias.is_contiguous()))):
      # decode-shaped product without a backward pass: one launch that streams w once
      return kernels.gemm_skinny(x2, w, bias=bias).view(*x.shape[:-1], N)
    if kernels.gemm_supported(M, N, K, x2, w) and w.is_contiguous():
      y = _LinearFn.apply(x2, w, w)
      y = y.view(*x.shape[:-1], N)
      if bias is not None:
        y = y + bias
      return y
  return ref.linear(x, w, bias)


# ------------------------------------------------------------------------------ rmsnorm
class _RMSNormFn(torch.autograd.Function):

  @staticmethod
  def forward(ctx, x2, w, eps, offset, holder):
    y, _, rstd = kernels.rmsnorm_fwd(x2, w, eps, offset)
    ctx.save_for_backward(x2, w, rstd)
    ctx.eps, ctx.offset, ctx.holder = eps, offset, holder
    return y

  @staticmethod
  def backward(ctx, dy):
    x2, w, rstd = ctx.saved_tensors
    mg = _main_grad(ctx.holder)
    if mg is not None:
      dx, _ = kernels.rmsnorm_bwd(x2, w, dy.contiguous(), rstd, ctx.eps, ctx.offset, dw_out=mg, dw_accumulate=True)
      return dx, None, None, None, None
    dx, dw = kernels.rmsnorm_bwd(x2, w, dy.contiguous(), rstd, ctx.eps, ctx.offset)
    return dx, dw.to(w.dtype), None, None, None


class _AddRMSNormFn(torch.autograd.Function):
  """(x, res) -> (norm(x + res), x + res): the residual add fused into the norm's read."""

  @staticmethod
  def forward(ctx, x2, res2, w, eps, offset, holder):
    y, s, rstd = kernels.rmsnorm_fwd(x2, w, eps, offset, residual=res2)
    ctx.save_for_backward(s, w, rstd)
    ctx.eps, ctx.offset, ctx.holder = eps, offset, holder
    return y, s

  @staticmethod
  def backward(ctx, dy, ds):
    s, w, rstd = ctx.saved_tensors
    mg = _main_grad(ctx.holder)
    dres = ds.contiguous() if ds is not None else None
    if mg is not None:
      dx, _ = kernels.rmsnorm_bwd(s, w, dy.contiguous(), rstd, ctx.eps, ctx.offset, dres=dres, dw_out=mg,
                                  dw_accumulate=True)
      dw = None
    else:
      dx, dwf = kernels.rmsnorm_bwd(s, w, dy.contiguous(), rstd, ctx.eps, ctx.offset, dres=dres)
      dw = dwf.to(w.dtype)
    return dx, dx, dw, None, None, None


def _norm_ok(x: torch.Tensor, w: torch.Tensor) -> bool:
  D = x.shape[-1]
  return _use_kernels(x) and w.dtype == bf16 and D % 8 == 0 and D <= 8192


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float = 1e-6, w_offset: float = 0.0) -> torch.Tensor:
  if _norm_ok(x, w):
    x2 = x.reshape(-1, x.shape[-1]).contiguous()
    return _RMSNormFn.apply(x2, w, eps, w_offset, w).view(x.shape)
  return ref.rms_norm(x, w, eps, w_offset)


def add_rms_norm(x: torch.Tensor, residual: torch.Tensor, w: torch.Tensor, eps: float = 1e-6,
                 w_offset: float = 0.0) -> Tuple[torch.Tensor, torch.Tensor]:
  """Returns (rms_norm(x + residual), x + residual)."""
  if _norm_ok(x, w):
    D = x.shape[-1]
    y, s = _AddRMSNormFn.apply(x.reshape(-1, D).contiguous(), residual.reshape(-1, D).contiguous(), w, eps,
                               w_offset, w)
    return y.view(x.shape), s.view(x.shape)
  s = x + residual
  return ref.rms_norm(s, w, eps, w_offset), s


# ------------------------------------------------------------------------------ qk-norm + rope
_rope_tables = {}
_bound = threading.local()     # per host thread: a rollout thread's bound must not leak into a trainer thread


def _position_bound() -> int:
  return getattr(_bound, "n", 0)


def set_position_bound(n: int) -> int:
  """Declares that every position this thread passes to `qk_norm_rope` is below `n` until further
  notice (0 = unknown). With a bound the rotary table is sized once and the per-call
  device-to-host read of `positions.max()` is skipped, which also makes the call capturable in
  a CUDA graph. A position that breaks the promise is clamped by the kernel and reported through
  the status word (bit 8). Returns the previous bound."""
  old = _position_bound()
  _bound.n = int(n)
  return old


def rope_table(head_dim: int, theta: float, max_pos: int, device, scale: float = 1.0) -> torch.Tensor:
  key = (head_dim, float(theta), float(scale), str(device))
  t = _rope_tables.get(key)
  if t is None or t.shape[0] < max_pos:
    n = max(4096, 1 << (max(1, max_pos) - 1).bit_length())
    t = kernels.rope_table(n, head_dim, theta, device, scale)
    _rope_tables[key] = t
  return t


class _QKNormRopeFn(torch.autograd.Function):

  @staticmethod
  def forward(ctx, qkv2, positions, table, n_q, n_k, H, wq, wk, eps, offset, hq, hk):
    out = kernels.qknorm_rope_fwd(qkv2, positions, table, n_q, n_k, H, wq, wk, eps, offset)
    ctx.save_for_backward(qkv2, positions, table, wq, wk)
    ctx.cfg = (n_q, n_k, H, eps, offset)
    ctx.hq, ctx.hk = hq, hk
    return out

  @staticmethod
  def backward(ctx, dy):
    qkv2, positions, table, wq, wk = ctx.saved_tensors
    n_q, n_k, H, eps, offset = ctx.cfg
    dx, dwq, dwk = kernels.qknorm_rope_bwd(qkv2, dy.contiguous(), positions, table, n_q, n_k, H, wq, wk, eps, offset)
    gq = gk = None
    if wq is not None:
      mq, mk = _main_grad(ctx.hq), _main_grad(ctx.hk)
      if mq is not None:
        mq.add_(dwq)
        mk.add_(dwk)
      else:
        gq, gk = dwq.to(wq.dtype), dwk.to(wk.dtype)
    return dx, None, None, None, None, None, gq, gk, None, None, None, None


def qk_norm_rope(qkv: torch.Tensor, positions: torch.Tensor, n_q: int, n_k: int, head_dim: int, theta: float,
                 wq: Optional[torch.Tensor] = None, wk: Optional[torch.Tensor] = None, eps: float = 1e-6,
                 w_offset: float = 0.0, rope_scale: float = 1.0, max_pos: int = 0) -> torch.Tensor:
  """qkv [..., (n_q + 2 n_k) * H] (q heads | k heads | v heads) -> same shape, with optional
  per-head RMSNorm on q and k (tunix/models/qwen3/model.py:531-554) followed by half-split
  rotary embedding; v is passed through."""
  lead = qkv.shape[:-1]
  if _use_kernels(qkv) and head_dim in (64, 128, 256):
    q2 = qkv.reshape(-1, qkv.shape[-1]).contiguous()
    pos = positions.reshape(-1).to(torch.int32)
    bound = _position_bound()
    table = rope_table(head_dim, theta, max_pos or bound or 4096, qkv.device, rope_scale)
    if max_pos == 0 and bound == 0 and table.shape[0] < 1 << 20:
      # positions are data; make sure the table covers them (rare: only beyond 4096 tokens)
      need = int(pos.max().item()) + 1 if pos.numel() else 1
      if need > table.shape[0]:
        table = rope_table(head_dim, theta, need, qkv.device, rope_scale)
    out = _QKNormRopeFn.apply(q2, pos, table, n_q, n_k, head_dim, wq, wk, eps, w_offset, wq, wk)
    return out.view(*lead, -1)
  x = qkv.reshape(*lead, n_q + 2 * n_k, head_dim)
  q, k, v = x[..., :n_q, :], x[..., n_q:n_q + n_k, :], x[..., n_q + n_k:, :]
  if wq is not None:
    q = ref.rms_norm(q, wq, eps, w_offset)
    k = ref.rms_norm(k, wk, eps, w_offset)
  q = ref.apply_rope(q, positions, theta, rope_scale)
  k = ref.apply_rope(k, positions, theta, rope_scale)
  return torch.cat([q, k, v], dim=-2).reshape(*lead, -1)


# ------------------------------------------------------------------------------ GLU
class _GLUFn(torch.autograd.Function):

  @staticmethod
  def forward(ctx, gu2, gelu):
    ctx.save_for_backward(gu2)
    ctx.gelu = gelu
    return kernels.glu_fwd(gu2, gelu)

  @staticmethod
  def backward(ctx, dout):
    (gu2,) = ctx.saved_tensors
    return kernels.glu_bwd(gu2, dout.contiguous(), ctx.gelu), None


def glu(gu: torch.Tensor, kind: str = "silu") -> torch.Tensor:
  """act(gate) * up with gu = [gate | up] along the last axis."""
  F2 = gu.shape[-1]
  if _use_kernels(gu) and (F2 // 2) % 8 == 0:
    out = _GLUFn.apply(gu.reshape(-1, F2).contiguous(), kind == "gelu")
    return out.view(*gu.shape[:-1], F2 // 2)
  return ref.glu(gu, kind)


# ------------------------------------------------------------------------------ embedding
class _EmbeddingFn(torch.autograd.Function):

  @staticmethod
  def forward(ctx, ids, table, scale, holder):
    ctx.save_for_backward(ids)
    ctx.scale, ctx.holder, ctx.shape = scale, holder, table.shape
    return kernels.embedding_fwd(ids, table, scale)

  @staticmethod
  def backward(ctx, dout):
    (ids,) = ctx.saved_tensors
    mg = _main_grad(ctx.holder)
    from . import _lib
    if _lib.deterministic():
      # sorted accumulation (index_put_ with accumulate sorts the indices on CUDA) instead of fp32 atomics
      g = mg if mg is not None else torch.zeros(ctx.shape, dtype=torch.float32, device=dout.device)
      g.index_put_((ids.long(),), dout.float() * ctx.scale, accumulate=True)
      return None, (None if mg is not None else g.to(dout.dtype)), None, None
    if mg is not None:
      kernels.embedding_bwd(ids, dout.contiguous(), mg, ctx.scale)
      return None, None, None, None
    g = torch.zeros(ctx.shape, dtype=torch.float32, device=dout.device)
    kernels.embedding_bwd(ids, dout.contiguous(), g, ctx.scale)
    return None, g.to(dout.dtype), None, None


def embedding(ids: torch.Tensor, table: torch.Tensor, scale: float = 1.0) -> torch.Tensor:
  if _use_kernels(table) and table.shape[1] % 8 == 0:
    out = _EmbeddingFn.apply(ids.reshape(-1), table, scale, table)
    return out.view(*ids.shape, table.shape[1])
  return ref.embedding(ids, table, scale)


# ------------------------------------------------------------------------------ attention
def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, mask: Optional[torch.Tensor] = None,
              causal: bool = False, scale: Optional[float] = None, softcap: float = 0.0) -> torch.Tensor:
  """GQA attention. q [B,T,N,H], k/v [B,S,K,H]; mask [B,T,S] bool or None.
  `causal=True` with mask=None means the plain lower-triangular mask (T == S)."""
  H = q.shape[-1]
  scale = (1.0 / math.sqrt(H)) if scale is None else scale
  if q.is_cuda and q.dtype in (bf16, torch.float16) and softcap == 0.0:
    from . import attention as _attn
    return _attn.attention_cuda(q, k, v, mask=mask, causal=causal, scale=scale)
  if mask is not None and not isinstance(mask, torch.Tensor):
    mask = mask.dense()          # a symbolic segment mask
  if mask is None and causal:
    T, S = q.shape[1], k.shape[1]
    mask = torch.ones(T, S, dtype=torch.bool, device=q.device).tril(S - T)[None].expand(q.shape[0], T, S)
  return ref.attention(q, k, v, mask, scale, softcap)


# ------------------------------------------------------------------------------ lm_head + log-softmax
_LOGITS_BUDGET_BYTES = 1 << 30   # size of one fp32 logits block kept live at a time


def _chunk_rows(T: int, V: int) -> int:
  rows = max(128, _LOGITS_BUDGET_BYTES // (4 * V))
  rows = (rows // 128) * 128
  return min(T, rows)


class _LinearLogprobFn(torch.autograd.Function):
  """Sequence-chunked lm_head -> selective log-softmax (tunix/rl/common.py:485-571 does the
  same with a rematerialised scan): the [T, V] logits are never resident, only one block."""

  @staticmethod
  def forward(ctx, h2, w, targets, inv_temp, softcap, want_entropy, holder):
    T, D = h2.shape
    V = w.shape[0]
    rows = _chunk_rows(T, V)
    logp = torch.empty(T, dtype=torch.float32, device=h2.device)
    lse = torch.empty(T, dtype=torch.float32, device=h2.device)
    ent = torch.empty(T, dtype=torch.float32, device=h2.device) if want_entropy else None
    buf = torch.empty((rows, V), dtype=torch.float32, device=h2.device)
    for s in range(0, T, rows):
      e = min(T, s + rows)
      lg = kernels.gemm(h2[s:e], w, out=buf[: e - s])
      lp, ls, en = kernels.logprob_fwd(lg, targets[s:e], inv_temp, softcap, want_entropy)
      logp[s:e], lse[s:e] = lp, ls
      if want_entropy:
        ent[s:e] = en
    ctx.save_for_backward(h2, w, targets, lse, ent)
    ctx.cfg = (inv_temp, softcap, rows)
    ctx.holder = holder
    if want_entropy:
      return logp, ent
    return logp, None

  @staticmethod
  def backward(ctx, g_logp, g_ent):
    h2, w, targets, lse, ent = ctx.saved_tensors
    inv_temp, softcap, rows = ctx.cfg
    T, D = h2.shape
    V = w.shape[0]
    need_dh, need_dw = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
    dh = torch.empty_like(h2) if need_dh else None
    mg = _main_grad(ctx.holder) if need_dw else None
    dw_acc = None
    if need_dw and mg is None:
      dw_acc = torch.zeros((V, D), dtype=torch.float32, device=h2.device)
    g_logp = g_logp.contiguous().float() if g_logp is not None else None
    g_ent = g_ent.contiguous().float() if g_ent is not None else None
    buf = torch.empty((rows, V), dtype=torch.float32, device=h2.device)
    dbuf = torch.empty((rows, V), dtype=bf16, device=h2.device)
    for s in range(0, T, rows):
      e = min(T, s + rows)
      lg = kernels.gemm(h2[s:e], w, out=buf[: e - s])
      dl = kernels.logprob_bwd(lg, targets[s:e], lse[s:e], ent[s:e] if ent is not None else None,
                               g_logp[s:e] if g_logp is not None else None,
                               g_ent[s:e] if g_ent is not None else None, inv_temp, softcap, out=dbuf[: e - s])
      if need_dh:
        kernels.gemm(dl, w, b_mn=True, out=dh[s:e])
      if need_dw:
        kernels.gemm(dl, h2[s:e], a_mn=True, b_mn=True, out=mg if mg is not None else dw_acc, accumulate=True)
    dw = None if (not need_dw or mg is not None) else dw_acc.to(w.dtype)
    return dh, dw, None, None, None, None, None


def linear_logprob(hidden: torch.Tensor, weight: torch.Tensor, targets: torch.Tensor, temperature: float = 1.0,
                   softcap: float = 0.0, want_entropy: bool = False):
  """Per-token log-probability (and entropy) of `targets` under softmax(hidden @ weight^T / T).

  hidden [..., D], weight [V, D], targets [...] -> (logp [...], entropy [...] or None), fp32.
  Shared by the trainer, the reference policy and the rollout sampler so that log-probs agree.
  """
  vp = getattr(weight, "vocab_parallel", None)
  if vp is not None:        # (group, first vocabulary row of this rank's slice): see ops/vocab_parallel.py
    from . import vocab_parallel
    return vocab_parallel.linear_logprob(hidden, weight, targets, vp[0], vp[1], temperature, softcap, want_entropy)
  lead = targets.shape
  D = hidden.shape[-1]
  V = weight.shape[0]
  inv_temp = 1.0 if temperature in (0.0, 1.0) else 1.0 / temperature
  if _use_kernels(hidden, weight) and weight.dtype == bf16 and V % 8 == 0 and D % 8 == 0 and weight.is_contiguous():
    h2 = hidden.reshape(-1, D).contiguous()
    T = h2.shape[0]
    pad = (-T) % 8
    tg = targets.reshape(-1)
    if pad:
      h2 = torch.cat([h2, h2.new_zeros(pad, D)], 0)
      tg = torch.cat([tg, tg.new_zeros(pad)], 0)
    lp, ent = _LinearLogprobFn.apply(h2, weight, tg, inv_temp, softcap, want_entropy, weight)
    lp = lp[:T].view(lead)
    ent = ent[:T].view(lead) if ent is not None else None
    return lp, ent
  lp, ent = ref.linear_logprob(hidden.reshape(-1, D), weight, targets.reshape(-1), temperature, softcap, want_entropy)
  return lp.view(lead), (ent.view(lead) if ent is not None else None)
