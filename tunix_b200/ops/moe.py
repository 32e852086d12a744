"""Grouped expert MLP for mixture-of-experts layers.

Two forms of the reference's three grouped matmuls (tunix/models/qwen3/model.py:975-995):

* `grouped_mlp(xs, counts, ...)`: rows sorted by expert, a Python loop of dense GEMM chains, one per
  expert (CPU, odd shapes, and the host-counted expert-parallel path).
* `padded_layout` + `grouped_mlp_padded`: the CUDA path. Every expert's rows are placed in a block
  padded with zero rows to a multiple of 128, the placement is computed on the device (no host
  round trip for the counts), and each of gate|up, down and their gradients is ONE launch of the
  grouped tcgen05 GEMM (`csrc/gemm_grouped.cu`) over all experts.
"""
from __future__ import annotations

import dataclasses
from typing import List, Optional

import torch

from . import _lib
from . import functional as F

bf16 = torch.bfloat16
TILE = 128


def grouped_mlp(xs: torch.Tensor, counts: List[int], gate_up: torch.Tensor, down: torch.Tensor, kind: str,
                first_expert: int = 0) -> torch.Tensor:
  outs = []
  start = 0
  for e, c in enumerate(counts):
    if c == 0:
      continue
    x = xs[start:start + c]
    h = F.glu(F.linear(x, gate_up[first_expert + e]), kind)
    outs.append(F.linear(h, down[first_expert + e]))
    start += c
  if not outs:
    return xs.new_zeros(xs.shape)
  return torch.cat(outs, dim=0)


# ------------------------------------------------------------------------------ padded layout
@dataclasses.dataclass
class PaddedLayout:
  """Where each routed row lives in the expert-major, 128-row-padded buffer."""
  rows: int                  # static size of the buffer: a bound that holds for any routing
  dest: torch.Tensor         # [n] int64: buffer row of routed row i (i = token * k + slot)
  offsets: torch.Tensor      # [E + 1] int32: first buffer row of each expert (multiples of 128)
  tile_expert: torch.Tensor  # [rows / 128] int32: expert of each row tile, -1 past the last block
  num_experts: int


def padded_rows(n: int, num_experts: int) -> int:
  """Buffer rows that fit n routed rows however they fall on the experts."""
  return (n + num_experts * (TILE - 1) + TILE - 1) // TILE * TILE


def count_rows(ids: torch.Tensor, num_experts: int) -> torch.Tensor:
  """Rows per expert without the device-to-host read that `torch.bincount` does to size its result."""
  return torch.zeros(num_experts, dtype=torch.long, device=ids.device).scatter_add_(
      0, ids.reshape(-1).long(), torch.ones(ids.numel(), dtype=torch.long, device=ids.device))


def padded_layout(expert_ids: torch.Tensor, num_experts: int, counts: Optional[torch.Tensor] = None,
                  rank_in_expert: Optional[torch.Tensor] = None) -> PaddedLayout:
  """expert_ids [n]: expert of every routed row. All device-side; nothing is read back."""
  n = expert_ids.numel()
  E = num_experts
  ids = expert_ids.reshape(-1).long()
  if counts is None:
    counts = count_rows(ids, E)
  padded = (counts + (TILE - 1)) // TILE * TILE
  offsets = torch.zeros(E + 1, dtype=torch.long, device=ids.device)
  offsets[1:] = torch.cumsum(padded, 0)
  if rank_in_expert is None:
    order = torch.argsort(ids, stable=True)
    start = torch.cumsum(counts, 0) - counts                     # first sorted position of each expert
    rank_sorted = torch.arange(n, device=ids.device) - start[ids[order]]
    rank_in_expert = torch.empty_like(rank_sorted).index_copy_(0, order, rank_sorted)
  dest = offsets[ids] + rank_in_expert
  rows = padded_rows(n, E)
  tile_start = torch.arange(rows // TILE, device=ids.device) * TILE
  te = torch.searchsorted(offsets[1:].contiguous(), tile_start, right=True)
  te = torch.where(tile_start < offsets[E], te, torch.full_like(te, -1))
  return PaddedLayout(rows, dest, offsets.int(), te.int(), E)


def grouped_supported(x: torch.Tensor, w: torch.Tensor) -> bool:
  """bf16 CUDA operands whose shapes the grouped kernel takes (`w` is [E, N, K])."""
  if not (x.is_cuda and x.dtype == bf16 and w.dtype == bf16 and w.dim() == 3 and w.is_contiguous()):
    return False
  _, N, K = w.shape
  return N % 64 == 0 and K % 8 == 0 and _lib.available()


def _call(mode, a, b, c, lay: PaddedLayout, N, K, E, accumulate=False):
  lib = _lib.require()
  rc = lib.tx_gemm_grouped_bf16(a.data_ptr(), b.data_ptr(), c.data_ptr(), lay.tile_expert.data_ptr(),
                                lay.offsets.data_ptr(), mode, lay.rows, N, K, E, a.stride(0),
                                b.stride(-2), c.stride(-2), int(c.dtype == torch.float32), int(accumulate), 1.0,
                                _lib.status_word(a.device).data_ptr(), _lib.stream_ptr())
  _lib.check_rc(rc, f"tx_gemm_grouped_bf16(mode={mode},R={lay.rows},N={N},K={K},E={E})")
  return c


class _GroupedLinear(torch.autograd.Function):
  """y[r] = x[r] @ w[expert(r)]^T over the padded layout."""

  @staticmethod
  def forward(ctx, x, w, lay, first_expert):
    E_all, N, K = w.shape
    E = lay.num_experts
    wv = w[first_expert:first_expert + E]
    y = torch.zeros((lay.rows, N), dtype=bf16, device=x.device)     # rows of unused tiles stay zero
    _call(0, x, wv, y, lay, N, K, E)
    ctx.save_for_backward(x, w)
    ctx.lay, ctx.first = lay, first_expert
    return y

  @staticmethod
  def backward(ctx, dy):
    x, w = ctx.saved_tensors
    lay, first = ctx.lay, ctx.first
    E_all, N, K = w.shape
    E = lay.num_experts
    dy = dy.contiguous()
    wv = w[first:first + E]
    dx = None
    if ctx.needs_input_grad[0]:
      # rows of unused tiles are never gathered; zero-fill so that they stay finite
      dx = torch.zeros((lay.rows, K), dtype=bf16, device=dy.device)
      _call(1, dy, wv, dx, lay, N, K, E)
    dw = None
    if ctx.needs_input_grad[1]:
      mg = getattr(w, "main_grad", None)
      if mg is not None:
        _call(2, dy, x, mg[first:first + E], lay, N, K, E, accumulate=True)
      else:
        dw = torch.zeros_like(w)
        _call(2, dy, x, dw[first:first + E], lay, N, K, E)
    return dx, dw, None, None


def grouped_linear(x: torch.Tensor, w: torch.Tensor, lay: PaddedLayout, first_expert: int = 0) -> torch.Tensor:
  return _GroupedLinear.apply(x.contiguous(), w, lay, first_expert)


def grouped_mlp_padded(x_pad: torch.Tensor, lay: PaddedLayout, gate_up: torch.Tensor, down: torch.Tensor, kind: str,
                       first_expert: int = 0) -> torch.Tensor:
  """x_pad [lay.rows, D] (padding rows zero) -> [lay.rows, D]; three grouped launches forward."""
  gu = grouped_linear(x_pad, gate_up, lay, first_expert)
  return grouped_linear(F.glu(gu, kind), down, lay, first_expert)


def scatter_rows(x2: torch.Tensor, token_of_row: torch.Tensor, lay: PaddedLayout) -> torch.Tensor:
  """Places token rows into the padded buffer (zero elsewhere); differentiable."""
  buf = torch.zeros((lay.rows, x2.shape[1]), dtype=x2.dtype, device=x2.device)
  return buf.index_copy(0, lay.dest, x2.index_select(0, token_of_row))


# Single-rank dispatch / combine on the row kernels of `csrc/moe_dispatch.cu` (the same kernels the expert-parallel
# path runs over peer memory, here with one "rank" whose buffer is local): one pass over the routed rows each way
# instead of index_select + index_copy and index_select + multiply + sum.
def _row_ptrs(buf: torch.Tensor):
  import ctypes
  return (ctypes.c_void_p * 1)(buf.data_ptr())


def _dispatch_rows(src: torch.Tensor, k: int, scale: Optional[torch.Tensor], dest32: torch.Tensor, zero_rank: torch.Tensor,
                   rows: int) -> torch.Tensor:
  D = src.shape[1]
  buf = torch.zeros((rows, D), dtype=bf16, device=src.device)
  rc = _lib.require().tx_moe_dispatch_rows(src.data_ptr(), src.stride(0), None, k,
                                           scale.data_ptr() if scale is not None else None, zero_rank.data_ptr(),
                                           dest32.data_ptr(), _row_ptrs(buf), 1, dest32.numel(), D, rows,
                                           _lib.status_word(src.device).data_ptr(), _lib.stream_ptr())
  _lib.check_rc(rc, "tx_moe_dispatch_rows")
  return buf


def _combine_rows(buf: torch.Tensor, weights: Optional[torch.Tensor], k: int, T: int, dest32: torch.Tensor,
                  zero_rank: torch.Tensor, keep_rows: bool):
  D = buf.shape[1]
  out = torch.empty((T, D), dtype=bf16, device=buf.device)
  gathered = torch.empty((T * k, D), dtype=bf16, device=buf.device) if keep_rows else None
  rc = _lib.require().tx_moe_combine_rows(_row_ptrs(buf), 1, zero_rank.data_ptr(), dest32.data_ptr(),
                                          weights.data_ptr() if weights is not None else None, k, out.data_ptr(),
                                          out.stride(0), gathered.data_ptr() if gathered is not None else None, T, D,
                                          buf.shape[0], _lib.status_word(buf.device).data_ptr(), _lib.stream_ptr())
  _lib.check_rc(rc, "tx_moe_combine_rows")
  return out, gathered


class _LocalDispatch(torch.autograd.Function):

  @staticmethod
  def forward(ctx, x2, dest32, zero_rank, rows, k):
    ctx.save_for_backward(dest32, zero_rank)
    ctx.k, ctx.T = k, x2.shape[0]
    return _dispatch_rows(x2, k, None, dest32, zero_rank, rows)

  @staticmethod
  def backward(ctx, dbuf):
    dest32, zero_rank = ctx.saved_tensors
    dx, _ = _combine_rows(dbuf.contiguous(), None, ctx.k, ctx.T, dest32, zero_rank, keep_rows=False)
    return dx, None, None, None, None


class _LocalCombine(torch.autograd.Function):

  @staticmethod
  def forward(ctx, y_pad, topv, dest32, zero_rank):
    T, k = topv.shape
    w = topv.reshape(-1).float().contiguous()
    out, gathered = _combine_rows(y_pad, w, k, T, dest32, zero_rank, keep_rows=True)
    ctx.save_for_backward(gathered, w, dest32, zero_rank)
    ctx.shape, ctx.rows = (T, k), y_pad.shape[0]
    return out

  @staticmethod
  def backward(ctx, dout):
    gathered, w, dest32, zero_rank = ctx.saved_tensors
    T, k = ctx.shape
    dout = dout.contiguous()
    dtopv = torch.einsum("tkd,td->tk", gathered.view(T, k, -1).float(), dout.float())
    return _dispatch_rows(dout, k, w, dest32, zero_rank, ctx.rows), dtopv, None, None


def moe_forward_padded(x2: torch.Tensor, topv: torch.Tensor, topi: torch.Tensor, gate_up: torch.Tensor,
                       down: torch.Tensor, kind: str) -> torch.Tensor:
  """Single-rank routed MLP: x2 [T, D], topv/topi [T, k] -> [T, D]."""
  T, k = topi.shape
  E = gate_up.shape[0]
  lay = padded_layout(topi.reshape(-1), E)
  if x2.shape[1] % 8 == 0 and k <= 16:
    dest32 = lay.dest.int()
    zero_rank = torch.zeros_like(dest32)
    x_pad = _LocalDispatch.apply(x2.contiguous(), dest32, zero_rank, lay.rows, k)
    y_pad = grouped_mlp_padded(x_pad, lay, gate_up, down, kind)
    return _LocalCombine.apply(y_pad, topv.float(), dest32, zero_rank)
  tok = torch.arange(T, device=x2.device).repeat_interleave(k)
  y_pad = grouped_mlp_padded(scatter_rows(x2, tok, lay), lay, gate_up, down, kind)
  ys = y_pad.index_select(0, lay.dest) * topv.reshape(-1, 1).to(y_pad.dtype)
  return ys.view(T, k, -1).sum(1)
