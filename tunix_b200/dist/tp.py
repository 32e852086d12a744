"""Megatron-style tensor parallelism for the decoder (dense layers).

`shard_model_tp(model, mesh, axis="tp")` returns this rank's slice of the model: query and kv
heads are split over the ranks of `axis` (rows of the fused qkv projection, columns of the
output projection), the MLP's hidden units likewise (rows of gate and of up, columns of down).
Embedding, norms and lm_head stay replicated. The two partial sums per layer (after `o_proj`
and after `down_proj`) are all-reduced; gradients flowing back into the replicated activations
are all-reduced where the forward was an identity (the f / g pair of Megatron-LM). The KV
cache (dense or paged) shrinks with the local kv-head count without further changes, and a
rollout engine on each rank samples identical tokens because the all-reduced logits are
bitwise equal on all ranks and sampling is keyed by (seed, step, row).

Reference behaviour: the `'tp'` mesh axis on heads and FFN hidden units
(tunix/models/qwen3/model.py:111-134); here the collectives are explicit NCCL all-reduces.
"""
from __future__ import annotations

import copy
from typing import Optional

import torch
import torch.distributed as dist


class _CopyToRegion(torch.autograd.Function):
  """Identity forward, all-reduce of the gradient backward (entry of a column-parallel layer)."""

  @staticmethod
  def forward(ctx, x, group):
    ctx.group = group
    return x

  @staticmethod
  def backward(ctx, g):
    g = g.contiguous()
    dist.all_reduce(g, group=ctx.group)
    return g, None


class _ReduceFromRegion(torch.autograd.Function):
  """All-reduce forward, identity backward (exit of a row-parallel layer)."""

  @staticmethod
  def forward(ctx, x, group):
    x = x.contiguous()
    dist.all_reduce(x, group=group)
    return x

  @staticmethod
  def backward(ctx, g):
    return g, None


class _ColumnEntry(torch.nn.Module):

  def __init__(self, inner: torch.nn.Module, group):
    super().__init__()
    self.inner, self.group = inner, group

  def forward(self, x, *a, **k):
    return self.inner(_CopyToRegion.apply(x, self.group), *a, **k)

  def __getattr__(self, name):
    try:
      return super().__getattr__(name)
    except AttributeError:
      return getattr(super().__getattr__("inner"), name)


class _RowExit(_ColumnEntry):

  def forward(self, x, *a, **k):
    return _ReduceFromRegion.apply(self.inner(x, *a, **k), self.group)


class FusedRowExit(torch.nn.Module):
  """Row-parallel projection whose all-reduce runs inside the GEMM epilogue (inference path).

  Every rank owns a zero-filled fp32 [max_rows, out] buffer in peer-mapped memory. A call zeroes the rows it
  needs, meets the other ranks at a device-side barrier, runs `tx_gemm_bf16_allreduce` - each output tile is
  added with fp32 atomics over NVLink into every rank's buffer - meets them again, and rounds its buffer to
  bf16. Two bounded barriers and three launches replace GEMM + NCCL all-reduce. With gradients enabled,
  on the CPU, or for rows beyond `max_rows` the call falls back to GEMM + all-reduce."""

  def __init__(self, inner: torch.nn.Module, group, symm, max_rows: int):
    super().__init__()
    self.inner, self.group, self.symm, self.max_rows = inner, group, symm, int(max_rows)
    self.out_dim = inner.out_dim
    name = f"tp_sum_{id(self)}"
    self.buf = symm.alloc(name, self.max_rows * self.out_dim, torch.float32)
    self._name = name

  def __getattr__(self, name):
    try:
      return super().__getattr__(name)
    except AttributeError:
      return getattr(super().__getattr__("inner"), name)

  def forward(self, x):
    lin = self.inner
    x2 = x.reshape(-1, x.shape[-1])
    M = x2.shape[0]
    from ..ops import _lib as _lib0
    fused = (not _lib0.deterministic() and not torch.is_grad_enabled() and x2.is_cuda and x2.dtype == torch.bfloat16 and M <= self.max_rows
             and M % 8 == 0 and lin.b is None and lin.quant is None and not len(lin.lora_a)
             and x2.stride(1) == 1 and x2.data_ptr() % 16 == 0)
    if not fused:
      return _ReduceFromRegion.apply(lin(x), self.group)
    from ..ops import _lib
    from . import symm as symm_lib
    lib = _lib.require()
    N = self.out_dim
    ws = self.buf[:M * N]
    ws.zero_()
    self.symm.barrier()                      # every rank's buffer is clean before anybody adds into it
    ptrs = symm_lib._ptr_array(self.symm.peer_ptrs[self._name])
    rc = lib.tx_gemm_bf16_allreduce(x2.data_ptr(), lin.w.data_ptr(), ptrs, self.symm.world, M, N, x2.shape[1],
                                    x2.stride(0), lin.w.stride(0), 0, 0, 1.0,
                                    _lib.status_word(x2.device).data_ptr(), _lib.stream_ptr())
    _lib.check_rc(rc, "tx_gemm_bf16_allreduce")
    self.symm.barrier()                      # every rank's partial sums have landed
    out = torch.empty((M, N), dtype=torch.bfloat16, device=x2.device)
    _lib.check_rc(lib.tx_f32_sum_to_bf16(ws.data_ptr(), out.data_ptr(), N, M, N, _lib.stream_ptr()),
                  "tx_f32_sum_to_bf16")
    return out.view(*x.shape[:-1], N)


class SkinnyExitContext:
  """Peer-mapped scratch shared by all in-kernel tensor-parallel exits of one model replica.

  `part`: this rank's partial sums, two parities of [max_rows, max_out] fp32 (a call writes parity
  `epoch & 1`; the peers read it while the next call already fills the other one). `flags`: one int per
  (rank, 128-column block) that the owner of a block of partial sums sets to the call number. `epoch` and
  `done` are private device counters that the kernel itself advances, so the calls replay inside CUDA graphs.
  The exits of a model run one after another on one stream and therefore share one context."""

  def __init__(self, group, device: torch.device, max_rows: int, max_out: int, symm=None):
    from ..ops import _lib
    from . import symm as symm_lib
    lib = _lib.require()
    self.symm = symm or symm_lib.SymmetricBuffers(group, device)
    self.n_ranks, self.rank = self.symm.world, self.symm.rank
    self.max_rows, self.max_out = int(max_rows), int(max_out)
    self.part_stride = self.max_rows * self.max_out
    self.flag_blocks = lib.tx_gemm_skinny_flag_blocks()
    if (self.max_out + 127) // 128 > self.flag_blocks:
      raise ValueError(f"tensor-parallel exit wider than {128 * self.flag_blocks} columns")
    part = self.symm.alloc("tp_skinny_part", 2 * self.part_stride, torch.float32)
    flags = self.symm.alloc("tp_skinny_flags", self.n_ranks * self.flag_blocks, torch.int32)
    part.zero_()
    flags.zero_()
    self.symm.rendezvous()
    self.part_ptrs = symm_lib._ptr_array(self.symm.peer_ptrs["tp_skinny_part"])
    self.flag_ptrs = symm_lib._ptr_array(self.symm.peer_ptrs["tp_skinny_flags"])
    self.epoch = torch.zeros(1, dtype=torch.int32, device=device)
    self.done = torch.zeros(1, dtype=torch.int32, device=device)
    self.wait_ms = self.symm.wait_limit_ms

  def fits(self, rows: int, out_dim: int) -> bool:
    return rows <= min(self.max_rows, 128) and out_dim <= self.max_out and rows * out_dim <= self.part_stride


class SkinnyRowExit(torch.nn.Module):
  """Row-parallel projection of a tensor-parallel group. Decode-shaped inputs (at most 128 rows, no
  gradient) run `tx_gemm_skinny` with its in-kernel all-reduce over peer memory (`SkinnyExitContext`);
  anything else is GEMM + library all-reduce, like `_RowExit`."""

  skinny_exit = True

  def __init__(self, inner: torch.nn.Module, group, ctx: SkinnyExitContext):
    super().__init__()
    self.inner, self.group, self.tp_exit = inner, group, ctx

  def __getattr__(self, name):
    try:
      return super().__getattr__(name)
    except AttributeError:
      return getattr(super().__getattr__("inner"), name)

  def forward(self, x):
    lin = self.inner
    x2 = x.reshape(-1, x.shape[-1])
    from ..ops import kernels
    if (not torch.is_grad_enabled() and self.tp_exit.fits(x2.shape[0], lin.out_dim) and lin.b is None
        and lin.quant is None and not lin._lora_active() and kernels.gemm_skinny_supported(x2, lin.w)):
      y = kernels.gemm_skinny(x2 if x2.is_contiguous() else x2.contiguous(), lin.w, tp=self.tp_exit)
      return y.view(*x.shape[:-1], lin.out_dim)
    return _ReduceFromRegion.apply(lin(x), self.group)


def _slice_rows(w: torch.Tensor, sections, tp: int, r: int) -> torch.Tensor:
  """Takes rank r's share of every row section (sizes in `sections`) of w."""
  parts, off = [], 0
  for n in sections:
    per = n // tp
    parts.append(w[off + r * per: off + (r + 1) * per])
    off += n
  return torch.cat(parts, dim=0).clone()


def shard_model_tp(model: torch.nn.Module, mesh, axis: str = "tp", fused_max_rows: int = 0,
                   shard_vocab: bool = False, skinny_exit: bool = False) -> torch.nn.Module:
  """Builds this rank's tensor-parallel slice from a full (replicated) model and returns it.
  `shard_vocab` also splits an untied lm_head by vocabulary rows: log-probs then go through
  `ops.vocab_parallel` (three numbers per token cross the ranks), full logits are all-gathered.
  `fused_max_rows > 0` (CUDA ranks on one NVLink domain) makes the two exits of every layer `FusedRowExit`s
  for up to that many token rows per call (decode and chunked prefill of a rollout engine).
  `skinny_exit` (CUDA ranks on one NVLink domain) makes them `SkinnyRowExit`s instead: decode steps of up to 128
  rows sum the ranks' partial products inside the skinny GEMM kernel over peer memory."""
  from ..models.transformer import Transformer
  tp, r = mesh.axis_size(axis), mesh.axis_index(axis)
  if tp == 1:
    return model
  group = mesh.group(axis)
  cfg = model.config
  if cfg.is_moe:
    raise NotImplementedError("tensor parallelism covers dense layers; shard experts with dist.moe")
  N, K, H, Fh = cfg.num_heads, cfg.num_kv_heads, cfg.head_dim, cfg.hidden_dim
  if N % tp or K % tp or Fh % tp:
    raise ValueError(f"heads {N}/{K} and hidden {Fh} must divide by tp={tp}")
  # q_pre_attn scaling depends on the full head geometry: freeze it before the head counts change
  local = cfg.replace(num_heads=N // tp, num_kv_heads=K // tp, hidden_dim=Fh // tp,
                      query_pre_attn_scalar=cfg.query_pre_attn_scalar)
  dev = next(model.parameters()).device
  out = Transformer(local, device=dev)
  src = dict(model.named_parameters())
  with torch.no_grad():
    for name, p in out.named_parameters():
      w = src[name].data
      if name.endswith("attn.qkv_proj.w") or name.endswith("attn.qkv_proj.b"):
        p.copy_(_slice_rows(w, (N * H, K * H, K * H), tp, r))
      elif name.endswith("attn.o_proj.w"):
        per = N * H // tp
        p.copy_(w[:, r * per:(r + 1) * per])
      elif name.endswith("mlp.gate_up_proj.w"):
        p.copy_(_slice_rows(w, (Fh, Fh), tp, r))
      elif name.endswith("mlp.down_proj.w"):
        per = Fh // tp
        p.copy_(w[:, r * per:(r + 1) * per])
      else:
        p.copy_(w)
  symm = None
  if skinny_exit and dev.type == "cuda":
    ctx = SkinnyExitContext(group, dev, 128, cfg.embed_dim)
    for layer in out.layers:
      layer.attn.qkv_proj = _ColumnEntry(layer.attn.qkv_proj, group)
      layer.mlp.gate_up_proj = _ColumnEntry(layer.mlp.gate_up_proj, group)
      layer.attn.o_proj = SkinnyRowExit(layer.attn.o_proj, group, ctx)
      layer.mlp.down_proj = SkinnyRowExit(layer.mlp.down_proj, group, ctx)
    out.tp_exit = ctx
    return _finish_tp(out, local, cfg, group, tp, r, shard_vocab)
  if fused_max_rows > 0 and dev.type == "cuda":
    from . import symm as symm_lib
    symm = symm_lib.SymmetricBuffers(group, dev)
  for layer in out.layers:
    layer.attn.qkv_proj = _ColumnEntry(layer.attn.qkv_proj, group)
    layer.mlp.gate_up_proj = _ColumnEntry(layer.mlp.gate_up_proj, group)
    if symm is not None:
      layer.attn.o_proj = FusedRowExit(layer.attn.o_proj, group, symm, fused_max_rows)
      layer.mlp.down_proj = FusedRowExit(layer.mlp.down_proj, group, symm, fused_max_rows)
    else:
      layer.attn.o_proj = _RowExit(layer.attn.o_proj, group)
      layer.mlp.down_proj = _RowExit(layer.mlp.down_proj, group)
  if symm is not None:
    symm.rendezvous()
    for layer in out.layers:
      layer.attn.o_proj.buf.zero_()
      layer.mlp.down_proj.buf.zero_()
    torch.cuda.synchronize(dev)
    dist.barrier(group=group)
  return _finish_tp(out, local, cfg, group, tp, r, shard_vocab)


def _finish_tp(out, local, cfg, group, tp: int, r: int, shard_vocab: bool):
  # the fused decoder-layer node bypasses the wrapped projections
  out.config = local.replace(fused_layers=False)
  for layer in out.layers:
    layer.cfg = out.config
  out.tp_group, out.tp_size, out.tp_rank = group, tp, r
  if shard_vocab and out.lm_head is not None and cfg.vocab_size % tp == 0:
    per = cfg.vocab_size // tp
    with torch.no_grad():
      out.lm_head.w.data = out.lm_head.w.data[r * per:(r + 1) * per].clone()
    out.lm_head.w.vocab_parallel = (group, r * per)
  return out
