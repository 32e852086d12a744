"""Plain-PyTorch statements of every hot op.

These are the oracle the CUDA kernels are tested against, and the execution path for CPU
tensors (unit tests, the fp32 plumbing configuration). They are differentiable through
ordinary autograd and make no assumption about dtype.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn.functional as F

# Value the attention scores take where the mask forbids attention
# (tunix/models/llama3/model.py:382-396 uses the same large negative constant).
K_MASK = -2.3819763e38


def linear(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
  return F.linear(x, w, bias)


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float, w_offset: float = 0.0) -> torch.Tensor:
  """fp32 `x * rsqrt(mean(x^2) + eps) * (w + w_offset)`; Gemma uses w_offset = 1
  (tunix/models/gemma/model.py:715-740), Llama/Qwen use 0 (tunix/models/llama3/model.py:273-297)."""
  xf = x.float()
  y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * (w.float() + w_offset)
  return y.to(x.dtype)


def rope_cos_sin(positions: torch.Tensor, head_dim: int, theta: float, scale: float = 1.0):
  half = head_dim // 2
  inv = 1.0 / (theta ** (torch.arange(half, device=positions.device, dtype=torch.float32) * 2.0 / head_dim))
  ang = positions.float()[..., None] / scale * inv
  return ang.cos(), ang.sin()


def apply_rope(x: torch.Tensor, positions: torch.Tensor, theta: float, scale: float = 1.0) -> torch.Tensor:
  """Half-split rotary embedding on x[..., T, heads, H] with positions[..., T]
  (tunix/models/qwen3/model.py:404-425)."""
  H = x.shape[-1]
  cos, sin = rope_cos_sin(positions, H, theta, scale)
  cos, sin = cos[..., None, :], sin[..., None, :]
  xf = x.float()
  x1, x2 = xf[..., : H // 2], xf[..., H // 2:]
  return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1).to(x.dtype)


def glu(gu: torch.Tensor, kind: str) -> torch.Tensor:
  """`act(gate) * up` for gu = [gate | up] on the last axis; kind in {"silu", "gelu"} (tanh GELU)."""
  g, u = gu.chunk(2, dim=-1)
  a = F.gelu(g.float(), approximate="tanh") if kind == "gelu" else F.silu(g.float())
  return (a * u.float()).to(gu.dtype)


def embedding(ids: torch.Tensor, table: torch.Tensor, scale: float = 1.0) -> torch.Tensor:
  out = F.embedding(ids, table)
  if scale != 1.0:
    out = (out.float() * scale).to(table.dtype)
  return out


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, mask: Optional[torch.Tensor], scale: float,
              softcap: float = 0.0) -> torch.Tensor:
  """Dense GQA attention. q [B,T,N,H], k/v [B,S,K,H], mask [B,T,S] bool (True = attend).
  fp32 scores and softmax (tunix/models/qwen3/model.py:674-686)."""
  B, T, N, H = q.shape
  K = k.shape[2]
  G = N // K
  qf = q.float().view(B, T, K, G, H) * scale
  s = torch.einsum("btkgh,bskh->bkgts", qf, k.float())
  if softcap > 0:
    s = torch.tanh(s / softcap) * softcap
  if mask is not None:
    s = torch.where(mask[:, None, None, :, :], s, torch.full_like(s, K_MASK))
  p = torch.softmax(s, dim=-1)
  o = torch.einsum("bkgts,bskh->btkgh", p, v.float())
  return o.reshape(B, T, N, H).to(q.dtype)


def selective_log_softmax(logits: torch.Tensor, targets: torch.Tensor, temperature: float = 1.0,
                          want_entropy: bool = False):
  """`logit[target] - logsumexp(logits)` in fp32 (tunix/rl/common.py:187-203), entropy optional."""
  z = logits.float()
  if temperature not in (0.0, 1.0):
    z = z / temperature
  lse = torch.logsumexp(z, dim=-1)
  lp = z.gather(-1, targets.long().unsqueeze(-1)).squeeze(-1) - lse
  ent = None
  if want_entropy:
    lsm = z - lse.unsqueeze(-1)
    ent = -(lsm.exp() * lsm).sum(-1)
  return lp, ent


def linear_logprob(hidden: torch.Tensor, weight: torch.Tensor, targets: torch.Tensor, temperature: float = 1.0,
                   softcap: float = 0.0, want_entropy: bool = False):
  """lm_head + selective log-softmax. hidden [T,D], weight [V,D], targets [T]."""
  logits = hidden.float() @ weight.float().t()
  if softcap > 0:
    logits = torch.tanh(logits / softcap) * softcap
  return selective_log_softmax(logits, targets, temperature, want_entropy)
