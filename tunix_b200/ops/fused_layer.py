"""A whole decoder layer as one autograd node with a hand-scheduled backward.

Ordinary per-op autograd keeps every GEMM input alive (normed activations, the GLU output) or,
with per-layer rematerialisation, replays the whole layer forward - a third more GEMM work.
This node keeps exactly the tensors that are expensive to rebuild (the rotated q|k|v, the
attention output with its log-sum-exp, the gate|up pre-activation, the two residual-stream
values and the per-row norm statistics) and rebuilds the cheap ones (RMSNorm outputs, the GLU
product) inside the backward. Per token and layer that is (2 + qkv + 1 + 2F/D) * D bf16 values
instead of roughly twice that, and no GEMM is ever recomputed.

Scope: the training fast path - CUDA bf16, causal attention over unpadded rows, dense SwiGLU /
GeGLU MLP, optional per-head q/k norm, no KV cache, no LoRA adapters, no biases. Everything else
runs the modular path in `models/transformer.py`, which computes the same function.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import attention as attn_ops
from . import flash as flash_lib
from . import kernels

bf16 = torch.bfloat16


def _mg(p):
  return getattr(p, "main_grad", None)


def _wgrad(dy2: torch.Tensor, x2: torch.Tensor, w: torch.Tensor):
  """dW[N,K] = dy^T x, accumulated into w.main_grad when present; returns the grad or None."""
  mg = _mg(w)
  if mg is not None:
    kernels.gemm(dy2, x2, a_mn=True, b_mn=True, out=mg, accumulate=True)
    return None
  return kernels.gemm(dy2, x2, a_mn=True, b_mn=True)


def _vec_grad(dw_fp32: torch.Tensor, w: torch.Tensor):
  mg = _mg(w)
  if mg is not None:
    mg.add_(dw_fp32)
    return None
  return dw_fp32.to(w.dtype)


class DecoderLayerFn(torch.autograd.Function):

  @staticmethod
  def forward(ctx, h, positions, table, w_in, w_qkv, w_o, w_post, w_gu, w_d, wq_norm, wk_norm, cfg,
              segments=None):
    B, T, D = h.shape
    N, K, H = cfg.num_heads, cfg.num_kv_heads, cfg.head_dim
    eps, off = cfg.norm_eps, cfg.norm_offset
    gelu = cfg.activation == "gelu"
    h2d = h.reshape(B * T, D)
    x1, _, rstd1 = kernels.rmsnorm_fwd(h2d, w_in, eps, off)
    qkv_pre = kernels.gemm(x1, w_qkv)
    del x1
    qkv = kernels.qknorm_rope_fwd(qkv_pre, positions, table, N, K, H, wq_norm, wk_norm, eps, off)
    if wq_norm is None:
      qkv_pre = None
    q4 = qkv.view(B, T, N + 2 * K, H)
    o, attn_ctx = attn_ops.flash_fwd(q4[:, :, :N], q4[:, :, N:N + K], q4[:, :, N + K:], causal=True,
                                     scale=cfg.attn_scale, segments=segments)
    o2 = o.reshape(B * T, N * H)
    a = kernels.gemm(o2, w_o)
    x2, h_mid, rstd2 = kernels.rmsnorm_fwd(a, w_post, eps, off, residual=h2d)
    del a
    gu = kernels.gemm(x2, w_gu)
    del x2
    act = kernels.glu_fwd(gu, gelu)
    # residual add in the down-projection epilogue: out = h_mid + act @ w_d^T
    out = h_mid.clone()
    kernels.gemm(act, w_d, out=out, accumulate=True)
    del act
    ctx.save_for_backward(h2d, positions, table, rstd1, qkv_pre, qkv, o2, h_mid, rstd2, gu, w_in, w_qkv, w_o,
                          w_post, w_gu, w_d, wq_norm, wk_norm)
    ctx.attn_ctx = attn_ctx
    ctx.cfg = cfg
    ctx.shape = (B, T, D)
    return out.view(B, T, D)

  @staticmethod
  def backward(ctx, dout):
    (h2d, positions, table, rstd1, qkv_pre, qkv, o2, h_mid, rstd2, gu, w_in, w_qkv, w_o, w_post, w_gu, w_d,
     wq_norm, wk_norm) = ctx.saved_tensors
    cfg = ctx.cfg
    B, T, D = ctx.shape
    N, K, H = cfg.num_heads, cfg.num_kv_heads, cfg.head_dim
    eps, off = cfg.norm_eps, cfg.norm_offset
    gelu = cfg.activation == "gelu"
    dout2 = dout.reshape(B * T, D).contiguous()

    # ---- MLP ------------------------------------------------------------------------
    act = kernels.glu_fwd(gu, gelu)                              # rebuilt, not stored
    g_wd = _wgrad(dout2, act, w_d)
    dact = kernels.gemm(dout2, w_d, b_mn=True)
    del act
    dgu = kernels.glu_bwd(gu, dact, gelu)
    del dact
    x2, _, _ = kernels.rmsnorm_fwd(h_mid, w_post, eps, off, want_rstd=False)   # rebuilt
    g_wgu = _wgrad(dgu, x2, w_gu)
    del x2
    dx2 = kernels.gemm(dgu, w_gu, b_mn=True)
    del dgu
    mg = _mg(w_post)
    dh_mid, dw_post = kernels.rmsnorm_bwd(h_mid, w_post, dx2, rstd2, eps, off, dres=dout2,
                                          dw_out=mg, dw_accumulate=mg is not None)
    g_wpost = None if mg is not None else dw_post.to(w_post.dtype)
    del dx2

    # ---- attention ----------------------------------------------------------------------
    g_wo = _wgrad(dh_mid, o2, w_o)
    do2 = kernels.gemm(dh_mid, w_o, b_mn=True)
    q4 = qkv.view(B, T, N + 2 * K, H)
    dqkv = torch.empty_like(qkv)
    d4 = dqkv.view(B, T, N + 2 * K, H)
    attn_ops.flash_bwd(do2.view(B, T, N, H), q4[:, :, :N], q4[:, :, N:N + K], q4[:, :, N + K:],
                       o2.view(B, T, N, H), ctx.attn_ctx, d4[:, :, :N], d4[:, :, N:N + K], d4[:, :, N + K:])
    del do2
    g_wq = g_wk = None
    if wq_norm is not None:
      dpre, dwq, dwk = kernels.qknorm_rope_bwd(qkv_pre, dqkv, positions, table, N, K, H, wq_norm, wk_norm, eps, off)
      g_wq, g_wk = _vec_grad(dwq, wq_norm), _vec_grad(dwk, wk_norm)
    else:
      dpre = kernels.qknorm_rope_fwd(dqkv, positions, table, N, K, H, None, None, eps, off, inverse=True)
    del dqkv
    x1, _, _ = kernels.rmsnorm_fwd(h2d, w_in, eps, off, want_rstd=False)        # rebuilt
    g_wqkv = _wgrad(dpre, x1, w_qkv)
    del x1
    dx1 = kernels.gemm(dpre, w_qkv, b_mn=True)
    del dpre
    mg = _mg(w_in)
    dh, dw_in = kernels.rmsnorm_bwd(h2d, w_in, dx1, rstd1, eps, off, dres=dh_mid, dw_out=mg,
                                    dw_accumulate=mg is not None)
    g_win = None if mg is not None else dw_in.to(w_in.dtype)
    ready = getattr(w_in, "grad_ready_hook", None)
    if ready is not None:
      ready()        # every weight gradient of this layer has been issued (a sharded store may start reducing them)
    return (dh.view(B, T, D), None, None, g_win, g_wqkv, g_wo, g_wpost, g_wgu, g_wd, g_wq, g_wk, None, None)


def eligible(layer, h: torch.Tensor, cache, attn_mask) -> bool:
  """True when `layer` (a models.transformer.DecoderLayer) can run as the fused node."""
  cfg = layer.cfg
  if not (h.is_cuda and h.dtype == bf16 and cache is None):
    return False
  if getattr(layer.attn, "sp_group", None) is not None or getattr(layer.attn, "tp_group", None) is not None:
    return False
  if attn_mask is not None:
    # packed rows run fused when the flash kernel takes the segment bounds (head_dim 128)
    if not (isinstance(attn_mask, attn_ops.SegmentMask) and cfg.head_dim == 128 and flash_lib._DISABLED is False):
      return False
  if cfg.is_moe or cfg.qkv_bias or cfg.use_post_attn_norm or cfg.use_post_ffw_norm or cfg.attn_logits_soft_cap:
    return False
  if cfg.sliding_window_size and layer.attn.attn_type.name == "LOCAL_SLIDING":
    return False
  if cfg.head_dim not in (64, 128, 256) or cfg.embed_dim % 8 or cfg.embed_dim > 8192:
    return False
  a, m = layer.attn, layer.mlp
  for lin in (a.qkv_proj, a.o_proj, m.gate_up_proj, m.down_proj):
    if len(lin.lora_a) or lin.quant is not None or lin.b is not None:
      return False
  if (h.shape[0] * h.shape[1]) % 8:
    return False
  return True


def run(layer, h: torch.Tensor, positions: torch.Tensor, attn_mask=None) -> torch.Tensor:
  from .functional import rope_table
  cfg = layer.cfg
  a, m = layer.attn, layer.mlp
  theta, rscale = a._theta_scale()
  pos = positions.reshape(-1).to(torch.int32)
  need = cfg.max_position or (int(pos.max().item()) + 1)
  table = rope_table(cfg.head_dim, theta, need, h.device, rscale)
  wq = a.q_norm.w if a.q_norm is not None else None
  wk = a.k_norm.w if a.k_norm is not None else None
  return DecoderLayerFn.apply(h.contiguous(), pos, table, layer.input_layernorm.w, a.qkv_proj.w, a.o_proj.w,
                              layer.post_attention_layernorm.w, m.gate_up_proj.w, m.down_proj.w, wq, wk, cfg,
                              attn_mask.bounds() if attn_mask is not None else None)
