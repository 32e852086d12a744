"""One decoder layer of a paged decode step in eight launches.

A decode step feeds at most 128 new tokens (one per running sequence) through every layer, so
each projection is a skinny product bound by streaming its weight once. The modular layer
spends about sixteen launches per layer on it (GEMM + split-K memset and conversion, separate
GLU, page write, residual adds). This path issues, per layer:

  1. RMSNorm                                            (`tx_rmsnorm_fwd`)
  2. q|k|v projection (+ bias)                          (`tx_gemm_skinny`)
  3. qk-norm + RoPE + KV page write                     (`tx_qknorm_rope_fwd` with slots)
  4. paged attention (+ split combine)                  (`tx_paged_decode_attn_tc`)
  5. output projection + residual add                   (`tx_gemm_skinny`, residual epilogue)
  6. RMSNorm
  7. gate|up projection with the gated activation       (`tx_gemm_skinny`, GLU epilogue)
  8. down projection + residual add                     (`tx_gemm_skinny`, residual epilogue)

Under tensor parallelism (`dist.tp.shard_model_tp(..., skinny_exit=True)`) steps 5 and 8 also sum
the ranks' partial products inside the same kernel over peer memory. The arithmetic per element
is that of the modular layer (fp32 accumulation, one rounding to bf16 per op boundary, the
residual added in fp32 before that rounding), so log-probs agree with the trainer's within the
tolerance the rollout tests state.
"""
from __future__ import annotations

import os

import torch

from . import kernels, paged
from . import functional as F


def _plain(lin) -> bool:
  """A projection this path can call directly: bf16 weight, no active LoRA adapter, no quantisation."""
  inner = getattr(lin, "inner", lin)
  return (getattr(inner, "quant", None) is None and not inner._lora_active() and inner.w.dtype == torch.bfloat16
          and inner.w.is_contiguous())


def eligible(layer, h: torch.Tensor, cache) -> bool:
  cfg = layer.cfg
  if torch.is_grad_enabled() or not h.is_cuda or h.dtype != torch.bfloat16:
    return False
  if cache is None or isinstance(cache, dict) or getattr(cache, "mode", None) != "decode":
    return False
  B, T, D = h.shape
  if T != 1 or B > 128 or cfg.is_moe or layer.post_attn_norm is not None or layer.post_ffw_norm is not None:
    return False
  if cfg.head_dim not in (64, 128, 256) or D % 8 or cfg.attn_logits_soft_cap or getattr(layer.attn, "sp_group", None):
    return False
  a, m = layer.attn, layer.mlp
  if not all(_plain(x) for x in (a.qkv_proj, a.o_proj, m.gate_up_proj, m.down_proj)):
    return False
  for lin in (a.o_proj, m.gate_up_proj, m.down_proj):
    if getattr(lin, "inner", lin).b is not None:
      return False
  # tensor-parallel exits must be the in-kernel ones; a library all-reduce exit takes the modular path
  for lin in (a.o_proj, m.down_proj):
    if hasattr(lin, "inner") and not getattr(lin, "skinny_exit", False):
      return False
  if layer.attn.attn_type.name == "LOCAL_SLIDING" and cfg.sliding_window_size:
    return False
  return True


def _w(lin) -> torch.Tensor:
  return getattr(lin, "inner", lin).w


# Above this many rows the plain products (q|k|v, o_proj, down) take the general GEMM: the skinny kernel's 128-row
# variant halves its ring depth and was measured slower there (31.7 / 29.6 / 64.5 us against 25.6 / 27.6 / 45.9 at
# 128 rows), while gate|up keeps it for the fused GLU. Tensor-parallel exits always use the skinny kernel, which
# carries the all-reduce.
_SKINNY_PLAIN_MAX_ROWS = int(os.environ.get("TUNIX_B200_SKINNY_PLAIN_MAX_ROWS", "64"))


def _project(x: torch.Tensor, w: torch.Tensor, *, bias=None, residual=None, tp=None) -> torch.Tensor:
  """x Wᵀ (+ bias) (+ residual) for a decode batch, on whichever kernel is faster at this row count."""
  rows = x.shape[0]
  if rows <= _SKINNY_PLAIN_MAX_ROWS:
    return kernels.gemm_skinny(x, w, bias=bias, residual=residual, tp=tp)
  if tp is not None:
    # a tensor-parallel exit stays on the skinny kernel (it carries the all-reduce) but runs in chunks of at most
    # 64 rows, the kernel's fast variant; the weight slice of a TP rank is re-read from L2 by the second chunk.
    # Every rank of the group sees the same row count, so all of them issue the same sequence of exits.
    out = torch.empty((rows, w.shape[0]), dtype=x.dtype, device=x.device)
    for lo in range(0, rows, _SKINNY_PLAIN_MAX_ROWS):
      hi = min(rows, lo + _SKINNY_PLAIN_MAX_ROWS)
      kernels.gemm_skinny(x[lo:hi], w, out=out[lo:hi], bias=bias, tp=tp,
                          residual=None if residual is None else residual[lo:hi])
    return out
  if residual is not None:
    out = residual.clone()
    kernels.gemm(x, w, out=out, accumulate=True)
    return out
  out = kernels.gemm(x, w)
  return out if bias is None else out.add_(bias)


def run(layer, h: torch.Tensor, positions: torch.Tensor, cache) -> torch.Tensor:
  """h [B, 1, D] -> [B, 1, D]; K/V of the new tokens are written into `cache`'s pages."""
  cfg = layer.cfg
  B, _, D = h.shape
  N, K, H = cfg.num_heads, cfg.num_kv_heads, cfg.head_dim
  a, m = layer.attn, layer.mlp
  h2 = h.reshape(B, D)
  if not h2.is_contiguous():
    h2 = h2.contiguous()
  x, _, _ = kernels.rmsnorm_fwd(h2, layer.input_layernorm.w, cfg.norm_eps, cfg.norm_offset, want_rstd=False)
  qkv_lin = getattr(a.qkv_proj, "inner", a.qkv_proj)
  qkv = _project(x, qkv_lin.w, bias=qkv_lin.b)
  theta, rscale = a._theta_scale()
  table = F.rope_table(H, theta, cfg.max_position or F._position_bound() or 4096, h.device, rscale)
  pos = positions.reshape(-1).to(torch.int32)
  qkv = kernels.qknorm_rope_fwd(qkv, pos, table, N, K, H, a.q_norm.w if a.q_norm is not None else None,
                                a.k_norm.w if a.k_norm is not None else None, cfg.norm_eps, cfg.norm_offset,
                                slots=cache.slots, k_pages=cache.k_pages, v_pages=cache.v_pages)
  q = qkv[:, :N * H].view(B, N, H)
  o = paged.paged_decode_attention(q, cache.k_pages, cache.v_pages, cache.block_tables, cache.seq_lens,
                                   cfg.attn_scale, cache.num_splits, cache.max_len)
  h_mid = _project(o.view(B, N * H), _w(a.o_proj), residual=h2, tp=getattr(a.o_proj, "tp_exit", None))
  x2, _, _ = kernels.rmsnorm_fwd(h_mid, layer.post_attention_layernorm.w, cfg.norm_eps, cfg.norm_offset,
                                 want_rstd=False)
  act = kernels.gemm_skinny(x2, _w(m.gate_up_proj), glu="gelu" if m.kind == "gelu" else "silu")
  out = _project(act, _w(m.down_proj), residual=h_mid, tp=getattr(m.down_proj, "tp_exit", None))
  return out.view(B, 1, D)
