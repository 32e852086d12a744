"""Raw (non-autograd) Python entry points of the sm_100a kernels.

Each function validates shapes/dtypes, allocates outputs with torch and launches the kernel
on the current stream. Autograd glue and the CPU oracle live in `functional.py`.
"""
from __future__ import annotations

import contextlib
import math
import os
import threading
from typing import Optional, Tuple

import torch

from . import _lib

bf16 = torch.bfloat16


def _p(t: Optional[torch.Tensor]) -> Optional[int]:
  return None if t is None else t.data_ptr()


def gemm_supported(M: int, N: int, K: int, *tensors: torch.Tensor) -> bool:
  """Shapes the tcgen05 GEMM accepts: bf16, 16-byte aligned rows (multiples of 8)."""
  if M <= 0 or N <= 0 or K <= 0 or N % 8 or K % 8 or M % 8:
    return False
  return all(t.dtype == bf16 and t.is_cuda and t.data_ptr() % 16 == 0 for t in tensors)


def gemm(a: torch.Tensor, b: torch.Tensor, *, a_mn: bool = False, b_mn: bool = False,
         out: Optional[torch.Tensor] = None, out_dtype: torch.dtype = bf16, accumulate: bool = False,
         alpha: float = 1.0, max_ctas: int = 0) -> torch.Tensor:
  """C[M,N] (+)= alpha * op(a) @ op(b)^T on the tcgen05 tensor cores.

  a: [M,K] (a_mn=False) or [K,M] (a_mn=True); b: [N,K] (b_mn=False) or [K,N] (b_mn=True).
  Both are 2-D bf16 with unit inner stride. `out` may be bf16 or fp32 and, with
  `accumulate`, is added to in the epilogue (fp32 gradient accumulation, residual adds).
  """
  assert a.dim() == 2 and b.dim() == 2 and a.stride(1) == 1 and b.stride(1) == 1
  if a_mn:
    K, M = a.shape
  else:
    M, K = a.shape
  if b_mn:
    Kb, N = b.shape
  else:
    N, Kb = b.shape
  assert K == Kb, f"inner dims differ: {K} vs {Kb}"
  if out is None:
    assert not accumulate
    out = torch.empty((M, N), dtype=out_dtype, device=a.device)
  assert out.shape == (M, N) and out.stride(1) == 1 and out.dtype in (bf16, torch.float32)
  lib = _lib.require()
  rc = lib.tx_gemm_bf16(a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K, a.stride(0), b.stride(0),
                        out.stride(0), int(a_mn), int(b_mn), int(out.dtype == torch.float32), int(accumulate),
                        float(alpha), _lib.status_word(a.device).data_ptr(), int(max_ctas), _lib.stream_ptr())
  _lib.check_rc(rc, f"tx_gemm_bf16(M={M},N={N},K={K},a_mn={a_mn},b_mn={b_mn})")
  return out


def rmsnorm_fwd(x: torch.Tensor, w: torch.Tensor, eps: float, w_offset: float = 0.0,
                residual: Optional[torch.Tensor] = None, want_rstd: bool = True):
  """Returns (y, summed_residual_or_None, rstd). x, residual: [T, D] bf16 contiguous."""
  T, D = x.shape
  y = torch.empty_like(x)
  s = torch.empty_like(x) if residual is not None else None
  rstd = torch.empty(T, dtype=torch.float32, device=x.device) if want_rstd else None
  rc = _lib.require().tx_rmsnorm_fwd(x.data_ptr(), _p(residual), w.data_ptr(), y.data_ptr(), _p(s), _p(rstd), T, D,
                                     float(eps), float(w_offset), _lib.stream_ptr())
  _lib.check_rc(rc, "tx_rmsnorm_fwd")
  return y, s, rstd


def rmsnorm_bwd(x, w, dy, rstd, eps, w_offset=0.0, dres=None, dw_out: Optional[torch.Tensor] = None,
                dw_accumulate: bool = False):
  """Returns (dx, dw fp32). `dres` is added into dx (gradient of the residual stream)."""
  T, D = x.shape
  lib = _lib.require()
  P = lib.tx_rmsnorm_bwd_partials(T)
  partial = torch.empty((P, D), dtype=torch.float32, device=x.device)
  dx = torch.empty_like(x)
  if dw_out is None:
    dw_out = torch.empty(D, dtype=torch.float32, device=x.device)
    dw_accumulate = False
  rc = lib.tx_rmsnorm_bwd(x.data_ptr(), w.data_ptr(), dy.data_ptr(), _p(rstd), _p(dres), dx.data_ptr(),
                          partial.data_ptr(), dw_out.data_ptr(), int(dw_accumulate), T, D, float(eps),
                          float(w_offset), _lib.stream_ptr())
  _lib.check_rc(rc, "tx_rmsnorm_bwd")
  return dx, dw_out


def qknorm_rope_fwd(x: torch.Tensor, positions: torch.Tensor, cos_sin: torch.Tensor, n_q: int, n_k: int,
                    head_dim: int, wq: Optional[torch.Tensor] = None, wk: Optional[torch.Tensor] = None,
                    eps: float = 1e-6, w_offset: float = 0.0, inverse: bool = False,
                    slots: Optional[torch.Tensor] = None, k_pages: Optional[torch.Tensor] = None,
                    v_pages: Optional[torch.Tensor] = None) -> torch.Tensor:
  """x: [T, n_total*H] bf16 (q heads, then k heads, then anything else, e.g. v). The first
  n_q + n_k heads get (optional per-head RMSNorm and) rotary embedding; the rest is copied.

  With `slots` (int64 [T], -1 = skip) the rotated keys and the values are also stored into row
  `slots[t]` of the paged cache tensors `k_pages` / `v_pages` ([pages, page, n_k, H]) in the same
  launch. A position outside the rotary table (`cos_sin.shape[0]` rows) is clamped and sets
  status bit 8 instead of reading out of range."""
  T, W = x.shape
  n_total = W // head_dim
  out = torch.empty_like(x)
  if slots is not None:
    assert slots.dtype == torch.int64 and k_pages.is_contiguous() and v_pages.is_contiguous()
  rc = _lib.require().tx_qknorm_rope_fwd(x.data_ptr(), out.data_ptr(), positions.data_ptr(), cos_sin.data_ptr(),
                                         _p(wq), _p(wk), None, T, n_total, n_q, n_q + n_k, head_dim, x.stride(0),
                                         out.stride(0), float(eps), float(w_offset), int(inverse),
                                         cos_sin.shape[0], _lib.status_word(x.device).data_ptr(), _p(slots),
                                         _p(k_pages), _p(v_pages), _lib.stream_ptr())
  _lib.check_rc(rc, "tx_qknorm_rope_fwd")
  return out


def qknorm_rope_bwd(x, dy, positions, cos_sin, n_q, n_k, head_dim, wq=None, wk=None, eps=1e-6, w_offset=0.0):
  """Returns (dx, dwq fp32 or None, dwk fp32 or None)."""
  T, W = x.shape
  n_total = W // head_dim
  dx = torch.empty_like(x)
  dwq = dwk = None
  if wq is not None:
    dwq = torch.zeros(head_dim, dtype=torch.float32, device=x.device)
    dwk = torch.zeros(head_dim, dtype=torch.float32, device=x.device)
  rc = _lib.require().tx_qknorm_rope_bwd(x.data_ptr(), dy.data_ptr(), dx.data_ptr(), positions.data_ptr(),
                                         cos_sin.data_ptr(), _p(wq), _p(wk), _p(dwq), _p(dwk), T, n_total, n_q,
                                         n_q + n_k, head_dim, x.stride(0), dy.stride(0), dx.stride(0), float(eps),
                                         float(w_offset), cos_sin.shape[0], _lib.status_word(x.device).data_ptr(),
                                         _lib.stream_ptr())
  _lib.check_rc(rc, "tx_qknorm_rope_bwd")
  return dx, dwq, dwk


def glu_fwd(gu: torch.Tensor, gelu: bool) -> torch.Tensor:
  T, F2 = gu.shape
  out = torch.empty((T, F2 // 2), dtype=gu.dtype, device=gu.device)
  _lib.check_rc(_lib.require().tx_glu_fwd(gu.data_ptr(), out.data_ptr(), T, F2 // 2, int(gelu), _lib.stream_ptr()),
                "tx_glu_fwd")
  return out


def glu_bwd(gu: torch.Tensor, dout: torch.Tensor, gelu: bool) -> torch.Tensor:
  T, F2 = gu.shape
  dgu = torch.empty_like(gu)
  _lib.check_rc(_lib.require().tx_glu_bwd(gu.data_ptr(), dout.data_ptr(), dgu.data_ptr(), T, F2 // 2, int(gelu),
                                          _lib.stream_ptr()), "tx_glu_bwd")
  return dgu


def embedding_fwd(ids: torch.Tensor, table: torch.Tensor, scale: float = 1.0) -> torch.Tensor:
  ids32 = ids.reshape(-1).to(torch.int32)
  V, D = table.shape
  out = torch.empty((ids32.numel(), D), dtype=table.dtype, device=table.device)
  _lib.check_rc(_lib.require().tx_embedding_fwd(ids32.data_ptr(), table.data_ptr(), out.data_ptr(), ids32.numel(),
                                                D, V, float(scale), _lib.stream_ptr()), "tx_embedding_fwd")
  return out


def embedding_bwd(ids: torch.Tensor, dout: torch.Tensor, grad_table: torch.Tensor, scale: float = 1.0) -> None:
  """grad_table (fp32 [V, D]) += scatter of dout rows."""
  ids32 = ids.reshape(-1).to(torch.int32)
  V, D = grad_table.shape
  _lib.check_rc(_lib.require().tx_embedding_bwd(ids32.data_ptr(), dout.data_ptr(), grad_table.data_ptr(),
                                                ids32.numel(), D, V, float(scale), _lib.stream_ptr()),
                "tx_embedding_bwd")


def adamw_step(master, m, v, grad, param_bf16, *, lr, beta1, beta2, eps, weight_decay, step: int,
               grad_scale: Optional[torch.Tensor] = None, zero_grad: bool = True) -> None:
  """Flat fused AdamW on fp32 master weights; refreshes the bf16 compute copy."""
  n = master.numel()
  bc1 = 1.0 - beta1 ** step
  bc2 = 1.0 - beta2 ** step
  if not master.is_cuda:      # the same update in plain PyTorch (CPU ranks of the multi-process tests)
    g = grad.float() * (float(grad_scale) if grad_scale is not None else 1.0)
    m.mul_(beta1).add_(g, alpha=1.0 - beta1)
    v.mul_(beta2).addcmul_(g, g, value=1.0 - beta2)
    upd = (m / bc1) / ((v / bc2).sqrt() + eps) + weight_decay * master
    master.sub_(lr * upd)
    if param_bf16 is not None:
      param_bf16.copy_(master)
    if zero_grad:
      grad.zero_()
    return
  _lib.check_rc(_lib.require().tx_adamw(master.data_ptr(), m.data_ptr(), v.data_ptr(), grad.data_ptr(),
                                        _p(param_bf16), n, float(lr), float(beta1), float(beta2), float(eps),
                                        float(weight_decay), float(bc1), float(bc2), _p(grad_scale),
                                        int(zero_grad), _lib.stream_ptr()), "tx_adamw")


_scratch = {}


def _partials(device) -> torch.Tensor:
  key = torch.device(device).index
  t = _scratch.get(key)
  if t is None:
    t = torch.empty(_lib.require().tx_sumsq_partials(), dtype=torch.float32, device=device)
    _scratch[key] = t
  return t


def sumsq(x: torch.Tensor, out: torch.Tensor, accumulate: bool = False) -> None:
  """out[0] (+)= sum(x**2) for a flat fp32 tensor, deterministic reduction order."""
  assert x.dtype == torch.float32 and x.is_contiguous()
  _lib.check_rc(_lib.require().tx_sumsq(x.data_ptr(), x.numel(), _partials(x.device).data_ptr(), out.data_ptr(),
                                        int(accumulate), _lib.stream_ptr()), "tx_sumsq")


def clip_scale(sumsq_t, inv_denom_t, max_norm: float, norm_out, scale_out) -> None:
  _lib.check_rc(_lib.require().tx_clip_scale(sumsq_t.data_ptr(), _p(inv_denom_t), float(max_norm or 0.0),
                                             norm_out.data_ptr(), scale_out.data_ptr(), _lib.stream_ptr()),
                "tx_clip_scale")


def logprob_fwd(logits: torch.Tensor, targets: torch.Tensor, inv_temp: float = 1.0, softcap: float = 0.0,
                want_entropy: bool = False, n_valid: Optional[int] = None):
  """logits [T, >=V] fp32/bf16 -> (logp[T], lse[T], entropy[T] or None), all fp32."""
  T = logits.shape[0]
  V = n_valid if n_valid is not None else logits.shape[1]
  dev = logits.device
  logp = torch.empty(T, dtype=torch.float32, device=dev)
  lse = torch.empty(T, dtype=torch.float32, device=dev)
  ent = torch.empty(T, dtype=torch.float32, device=dev) if want_entropy else None
  tg = targets.to(torch.int32)
  _lib.check_rc(_lib.require().tx_logprob_fwd(logits.data_ptr(), int(logits.dtype == torch.float32), logits.stride(0),
                                              tg.data_ptr(), logp.data_ptr(), lse.data_ptr(), _p(ent), T, V,
                                              float(inv_temp), float(softcap), _lib.stream_ptr()), "tx_logprob_fwd")
  return logp, lse, ent


def logprob_bwd(logits, targets, lse, entropy, g_logp, g_ent, inv_temp=1.0, softcap=0.0, n_valid=None,
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
  """Returns bf16 dlogits [T, V_pad] where V_pad = logits.shape[1]."""
  T, V_pad = logits.shape
  V = n_valid if n_valid is not None else V_pad
  if out is None:
    out = torch.empty((T, V_pad), dtype=bf16, device=logits.device)
  tg = targets.to(torch.int32)
  _lib.check_rc(_lib.require().tx_logprob_bwd(logits.data_ptr(), int(logits.dtype == torch.float32), logits.stride(0),
                                              tg.data_ptr(), lse.data_ptr(), _p(entropy), _p(g_logp), _p(g_ent),
                                              out.data_ptr(), out.stride(0), T, V, V_pad, float(inv_temp),
                                              float(softcap), _lib.stream_ptr()), "tx_logprob_bwd")
  return out


def rope_table(max_pos: int, head_dim: int, theta: float, device, scale: float = 1.0) -> torch.Tensor:
  """[max_pos, head_dim] fp32 = [cos(H/2) | sin(H/2)], timescale theta^(2i/H)."""
  half = head_dim // 2
  inv = 1.0 / (theta ** (torch.arange(half, dtype=torch.float64) * 2.0 / head_dim))
  ang = torch.arange(max_pos, dtype=torch.float64)[:, None] / scale * inv[None, :]
  return torch.cat([ang.cos(), ang.sin()], dim=-1).to(torch.float32).to(device)


def gemm_allgather_b(a: torch.Tensor, shard_ptrs, rank: int, shard_rows: int, stage: torch.Tensor,
                     slab_count: torch.Tensor, *, ldb: Optional[int] = None, out: Optional[torch.Tensor] = None,
                     out_dtype: torch.dtype = bf16, accumulate: bool = False, alpha: float = 1.0,
                     wait_limit_ms: int = 2000) -> torch.Tensor:
  """C = a @ W^T with W [N, K] row-sharded over len(shard_ptrs) ranks: the all-gather of W runs inside the GEMM
  kernel (`csrc/gemm_allgather.cu`). `shard_ptrs[r]` is the device address of rank r's [shard_rows, K] block
  (peer-mapped; entry `rank` is local), `stage` a local [N, K] bf16 scratch and `slab_count` an int32 [N / 128]
  scratch. Every rank's shard must be final before any rank calls this."""
  import ctypes
  M, K = a.shape
  world = len(shard_ptrs)
  N = shard_rows * world
  if out is None:
    out = torch.empty((M, N), dtype=out_dtype, device=a.device)
  arr = (ctypes.c_void_p * world)(*[int(x) for x in shard_ptrs])
  rc = _lib.require().tx_gemm_bf16_allgather_b(
      a.data_ptr(), arr, world, rank, stage.data_ptr(), slab_count.data_ptr(), out.data_ptr(), M, N, K, a.stride(0),
      int(ldb or K), out.stride(0), int(out.dtype == torch.float32), int(accumulate), float(alpha), int(wait_limit_ms),
      _lib.status_word(a.device).data_ptr(), _lib.stream_ptr())
  _lib.check_rc(rc, f"tx_gemm_bf16_allgather_b(M={M},N={N},K={K},world={world})")
  return out


# ------------------------------------------------------------------------------ skinny (decode) GEMM
_SKINNY = os.environ.get("TUNIX_B200_SKINNY", "1") != "0"     # 0: decode products take the general GEMM (A/B runs)


_fixed_order = threading.local()


@contextlib.contextmanager
def fixed_reduction_order():
  """Within the block, skinny GEMMs of this thread reduce every output in one fixed order (no split of K over
  CTAs), as in the package-wide deterministic mode: computations that are replicated on several ranks and must
  agree bit for bit (the lm_head of a tensor-parallel rollout group) use it."""
  old = getattr(_fixed_order, "on", False)
  _fixed_order.on = True
  try:
    yield
  finally:
    _fixed_order.on = old


def gemm_skinny_supported(x2: torch.Tensor, w: torch.Tensor, glu: bool = False) -> bool:
  """At most 128 activation rows, bf16, 16-byte aligned rows, output width a multiple of 8."""
  if not _SKINNY or not (x2.is_cuda and x2.dtype == bf16 and w.dtype == bf16 and x2.dim() == 2 and w.dim() == 2):
    return False
  M, K = x2.shape
  N = w.shape[0] // 2 if glu else w.shape[0]
  return (0 < M <= 128 and w.shape[1] == K and K % 8 == 0 and N % 8 == 0 and x2.stride(1) == 1 and w.stride(1) == 1
          and x2.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and x2.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gemm_skinny(x: torch.Tensor, w: torch.Tensor, *, out: Optional[torch.Tensor] = None, glu: Optional[str] = None,
                residual: Optional[torch.Tensor] = None, bias: Optional[torch.Tensor] = None, alpha: float = 1.0,
                max_ctas: int = 0, tp=None) -> torch.Tensor:
  """y[M, N] = epilogue(alpha * x[M, K] @ w[N, K]^T) for M <= 128 in one launch that streams `w` once
  (`csrc/gemm_skinny.cu`: swapped operands, split-K over thread-block clusters with the partial sums
  exchanged through distributed shared memory; no workspace).

  glu: None | "silu" | "gelu" - `w` is then [gate rows | up rows] ([2N, K]) and y = act(x gate^T) * (x up^T).
  residual: [M, N] added to the product (may be `out` itself). bias: [N].
  tp: a `dist.tp.SkinnyExit`-like object with `n_ranks, rank, part_ptrs, flag_ptrs, part_stride, epoch, done,
  wait_ms`: the partial products of a tensor-parallel group are summed inside the kernel over peer memory.
  """
  M, K = x.shape
  N = w.shape[0] // 2 if glu else w.shape[0]
  if out is None:
    out = torch.empty((M, N), dtype=bf16, device=x.device)
  assert out.shape == (M, N) and out.dtype == bf16 and out.stride(1) == 1
  lib = _lib.require()
  g = {None: 0, "silu": 1, "gelu": 2}[glu]
  if tp is None:
    n_ranks, rank, parts, flags, stride, epoch, done, wait_ms = 1, 0, None, None, 0, None, None, 0
  else:
    n_ranks, rank, parts, flags = tp.n_ranks, tp.rank, tp.part_ptrs, tp.flag_ptrs
    stride, epoch, done, wait_ms = tp.part_stride, tp.epoch.data_ptr(), tp.done.data_ptr(), tp.wait_ms
  rc = lib.tx_gemm_skinny(x.data_ptr(), w.data_ptr(), out.data_ptr(), _p(residual), _p(bias), M, N, K, x.stride(0),
                          w.stride(0), out.stride(0), residual.stride(0) if residual is not None else 0, float(alpha),
                          g, int(_lib.deterministic() or getattr(_fixed_order, "on", False)), _lib.status_word(x.device).data_ptr(), int(max_ctas), n_ranks, rank, parts, flags, stride,
                          epoch, done, wait_ms, _lib.stream_ptr())
  _lib.check_rc(rc, f"tx_gemm_skinny(M={M},N={N},K={K},glu={glu})")
  return out
