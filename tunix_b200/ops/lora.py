"""Fused LoRA linear: y = x Wᵀ + Σᵢ sᵢ·(x Aᵢᵀ) Bᵢᵀ on output slice i, as one tensor-core pass.

The low-rank update is folded into the base GEMM as extra reduction columns: with
t = [s₁·x A₁ᵀ | s₂·x A₂ᵀ | …] (shape [T, R], R = Σ rᵢ) and B̂ the block-diagonal matrix of
the Bᵢ ([out, R]), y = [x | t] · [W | B̂]ᵀ. `tx_gemm_bf16_dual` walks the K blocks of (x, W) and then
those of (t, B̂) into the same TMEM accumulator, so the adapter costs one extra k-block per tile and
no extra pass over y. The backward uses the same trick for dx = dy W + (s·dy B̂) Â and three small
GEMMs for dA, dB (only the adapters train; W is frozen).

Reference semantics: tunix applies qwix LoRA as `W + A·B·alpha/rank`
(tunix/models/safetensors_saver.py:90-112); the unfused restatement is `models.transformer.Linear`.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch

from . import _lib, kernels

bf16 = torch.bfloat16
Adapter = Tuple[torch.Tensor, torch.Tensor, float, int, int]      # (A [r, in], B [hi - lo, r], scale, lo, hi)


def gemm_dual(a, b, a2, b2, *, b_mn: bool = False, out: Optional[torch.Tensor] = None, alpha: float = 1.0):
  """C = alpha * (a @ op(b)ᵀ + a2 @ op(b2)ᵀ); a [M,K], a2 [M,K2]; b [N,K] (or [K,N] with b_mn), b2 likewise."""
  M, K = a.shape
  K2 = a2.shape[1]
  N = b.shape[1] if b_mn else b.shape[0]
  if out is None:
    out = torch.empty((M, N), dtype=bf16, device=a.device)
  rc = _lib.require().tx_gemm_bf16_dual(
      a.data_ptr(), b.data_ptr(), a2.data_ptr(), b2.data_ptr(), out.data_ptr(), M, N, K, K2, a.stride(0), b.stride(0),
      a2.stride(0), b2.stride(0), out.stride(0), 0, int(b_mn), int(out.dtype == torch.float32), 0, float(alpha),
      _lib.status_word(a.device).data_ptr(), 0, _lib.stream_ptr())
  _lib.check_rc(rc, f"tx_gemm_bf16_dual(M={M},N={N},K={K},K2={K2})")
  return out


def supported(x2: torch.Tensor, w: torch.Tensor, adapters: Sequence[Adapter]) -> bool:
  if not (x2.is_cuda and x2.dtype == bf16 and w.dtype == bf16 and _lib.available()) or w.requires_grad:
    return False
  T, K = x2.shape
  R = sum(a.shape[0] for a, *_ in adapters)
  if T % 8 or K % 8 or w.shape[0] % 8 or R % 8 or R == 0 or x2.stride(1) != 1 or x2.data_ptr() % 16:
    return False
  return all(a.dtype == bf16 and b.dtype == bf16 and a.shape[0] % 8 == 0 for a, b, *_ in adapters)


def _stack(adapters: Sequence[Adapter], out_dim: int, device):
  a_cat = torch.cat([a for a, *_ in adapters], dim=0).contiguous()             # [R, in]
  R = a_cat.shape[0]
  b_hat = torch.zeros((out_dim, R), dtype=bf16, device=device)
  scale = torch.empty(R, dtype=torch.float32, device=device)
  off = 0
  spans = []
  for a, b, s, lo, hi in adapters:
    r = a.shape[0]
    b_hat[lo:hi, off:off + r] = b
    scale[off:off + r] = s
    spans.append((off, r, lo, hi))
    off += r
  return a_cat, b_hat, scale, spans


class _FusedLoraLinear(torch.autograd.Function):

  @staticmethod
  def forward(ctx, x2, w, spec, *ab):
    adapters = [(ab[2 * i], ab[2 * i + 1]) + spec[i] for i in range(len(spec))]
    a_cat, b_hat, scale, spans = _stack(adapters, w.shape[0], x2.device)
    t = kernels.gemm(x2, a_cat, out_dtype=torch.float32)                       # [T, R] = x Âᵀ
    t_s = (t * scale).to(bf16)
    y = gemm_dual(x2, w, t_s, b_hat)
    ctx.save_for_backward(x2, w, a_cat, b_hat, scale, t_s)
    ctx.spans = spans
    return y

  @staticmethod
  def backward(ctx, dy):
    x2, w, a_cat, b_hat, scale, t_s = ctx.saved_tensors
    dy = dy.contiguous()
    u = kernels.gemm(dy, b_hat, b_mn=True, out_dtype=torch.float32)            # dy B̂ [T, R]
    u_s = (u * scale).to(bf16)
    dx = gemm_dual(dy, w, u_s, a_cat, b_mn=True) if ctx.needs_input_grad[0] else None
    d_a = kernels.gemm(u_s, x2, a_mn=True, b_mn=True, out_dtype=torch.float32)  # u_sᵀ x [R, in]
    d_b = kernels.gemm(dy, t_s, a_mn=True, b_mn=True, out_dtype=torch.float32)  # dyᵀ t_s [out, R]
    grads: List[Optional[torch.Tensor]] = []
    for off, r, lo, hi in ctx.spans:
      grads.append(d_a[off:off + r].to(bf16))
      grads.append(d_b[lo:hi, off:off + r].to(bf16))
    return (dx, None, None, *grads)


def fused_lora_linear(x: torch.Tensor, w: torch.Tensor, adapters: Sequence[Adapter]) -> torch.Tensor:
  """x [..., in] -> [..., out]; `adapters` as documented above. Call `supported` first."""
  x2 = x.reshape(-1, x.shape[-1])
  spec = tuple((float(s), int(lo), int(hi)) for _, _, s, lo, hi in adapters)
  flat = []
  for a, b, *_ in adapters:
    flat += [a, b]
  y = _FusedLoraLinear.apply(x2, w, spec, *flat)
  return y.view(*x.shape[:-1], w.shape[0])
