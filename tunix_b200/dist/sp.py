"""Sequence parallelism: activations sharded along the sequence over one mesh axis, attention over keys and
values fetched from the ranks that own them (the reference's `'sp'` axis keeps K/V whole per shard and shards
only the queries; it has no ring or Ulysses variant - tunix/models/qwen3/model.py:576-672,
tunix/sft/sharding_utils.py).

Layouts. A row of L tokens is cut into chunks; a rank holds one or two of them:

  * `contiguous`: W chunks, rank r holds chunk r. Attention is causal, so rank r needs keys [0, (r + 1) T): the
    last rank does W times the attention work of the first.
  * `zigzag`: 2 W chunks, rank r holds chunks r and 2 W - 1 - r. Its two query chunks need r + 1 and 2 W - r key
    chunks - 2 W + 1 in total on EVERY rank, so the attention work is balanced.

For each held chunk the queries are the last rows of a key prefix, which is exactly the rectangular causal
case the flash kernels implement (queries aligned to the end of the keys). Everything outside attention is
per token and needs no communication; parameter gradients are partial sums over the sequence shards and are
reduced over the axis like data-parallel gradients.

Transport. On CUDA with bf16 activations the stacked K|V chunk of every rank sits in a peer-mapped buffer and
each rank PULLS exactly the chunks of its prefix over NVLink with the 2-D peer copy kernel
(`tx_peer_copy_2d`): no rank receives keys it will mask away, and there is one device-side barrier (bounded
wait) per attention call instead of a collective. The backward runs the other way: every rank publishes the
gradient of its prefix, and the owner of a chunk pulls and sums the pieces of the ranks that used it. On CPU
(gloo) and for other dtypes the same layout runs on `all_gather` / `all_reduce`.
"""
from __future__ import annotations

import os
from typing import Dict, List, Sequence, Tuple

import torch
import torch.distributed as dist

LAYOUTS = ("contiguous", "zigzag")
_PEER = os.environ.get("TUNIX_B200_SP_PEER", "1") != "0"


class Layout:
  """Which chunks of the sequence a rank of the axis holds."""

  def __init__(self, world: int, kind: str = "contiguous"):
    if kind not in LAYOUTS:
      raise ValueError(f"sequence-parallel layout must be one of {LAYOUTS}, got {kind!r}")
    self.world, self.kind = world, kind
    self.num_chunks = world if kind == "contiguous" else 2 * world
    self.per_rank = self.num_chunks // world

  def chunks(self, rank: int) -> Tuple[int, ...]:
    return (rank,) if self.kind == "contiguous" else (rank, self.num_chunks - 1 - rank)

  def owner(self, chunk: int) -> Tuple[int, int]:
    """(rank, slot within that rank's local rows) of a chunk."""
    if self.kind == "contiguous" or chunk < self.world:
      return chunk, 0
    return self.num_chunks - 1 - chunk, 1

  def users(self, chunk: int) -> List[int]:
    """Ranks whose key prefix contains `chunk`."""
    return [r for r in range(self.world) if max(self.chunks(r)) >= chunk]


# ------------------------------------------------------------------ peer-mapped transport
class _PeerState:
  """Peer-mapped staging buffers of one (group, device): two forward and two backward buffers used in
  alternation, so one barrier per call is enough - a buffer is rewritten two calls later, after every rank
  has passed the barrier of the call in between, which it enters only once its own pulls are done."""

  def __init__(self, group, device):
    from . import symm
    self.sb = symm.SymmetricBuffers(group, device)
    self.sb.rendezvous()
    self.cap = {"x": 0, "g": 0}
    self.gen = {"x": 0, "g": 0}
    self.calls = {"x": 0, "g": 0}

  def buffer(self, kind: str, numel: int) -> torch.Tensor:
    if numel > self.cap[kind]:
      self.gen[kind] += 1
      for p in (0, 1):
        self.sb.alloc(f"sp_{kind}{p}_{self.gen[kind]}", numel, torch.bfloat16)
      self.sb.rendezvous()            # collective: every rank grows at the same call, shapes being equal
      self.cap[kind] = numel
    self.calls[kind] += 1
    return self.sb.tensors[f"sp_{kind}{self.calls[kind] & 1}_{self.gen[kind]}"][:numel]


_peer_states: Dict[Tuple[int, int], _PeerState] = {}


def _peer_state(group, device) -> _PeerState:
  key = (id(group), device.index if device.index is not None else torch.cuda.current_device())
  st = _peer_states.get(key)
  if st is None:
    st = _peer_states[key] = _PeerState(group, device)
  return st


def _use_peer(x: torch.Tensor, group) -> bool:
  return _PEER and x.is_cuda and x.dtype == torch.bfloat16 and dist.get_backend(group) == "nccl"


class _PrefixGather(torch.autograd.Function):
  """x [B, slots * Tc, F] (this rank's chunks) -> [B, (cmax + 1) * Tc, F]: the key prefix of the rank's last
  chunk in global order. Backward: every chunk's owner receives the sum of the gradients of its users."""

  @staticmethod
  def forward(ctx, x, group, layout: Layout):
    rank = dist.get_rank(group)
    held = layout.chunks(rank)
    B, T, F = x.shape
    Tc = T // len(held)
    cmax = max(held)
    ctx.group, ctx.layout, ctx.rank, ctx.dims = group, layout, rank, (B, Tc, F)
    ctx.peer = _use_peer(x, group)
    x = x.contiguous()
    out = torch.empty(B, (cmax + 1) * Tc, F, dtype=x.dtype, device=x.device)
    if ctx.peer:
      st = _peer_state(group, x.device)
      mine = st.buffer("x", x.numel())
      mine.copy_(x.reshape(-1))
      st.sb.barrier()
      ptrs = st.sb.ptrs_for(mine)
      o2 = out.view(B, -1)
      for c in range(cmax + 1):
        owner, slot = layout.owner(c)
        dst = o2[:, c * Tc * F:(c + 1) * Tc * F]
        if owner == rank:
          dst.copy_(x.view(B, -1)[:, slot * Tc * F:(slot + 1) * Tc * F])
        else:
          st.sb.peer_copy_2d(ptrs[owner] + 2 * slot * Tc * F, dst, B, Tc * F, T * F)
      return out
    parts = [torch.empty_like(x) for _ in range(layout.world)]
    dist.all_gather(parts, x, group=group)
    for c in range(cmax + 1):
      owner, slot = layout.owner(c)
      out[:, c * Tc:(c + 1) * Tc] = parts[owner][:, slot * Tc:(slot + 1) * Tc]
    return out

  @staticmethod
  def backward(ctx, grad):
    layout, rank, group = ctx.layout, ctx.rank, ctx.group
    B, Tc, F = ctx.dims
    held = layout.chunks(rank)
    n_all = layout.num_chunks
    grad = grad.contiguous()
    if ctx.peer:
      st = _peer_state(group, grad.device)
      ld = n_all * Tc * F                          # every rank publishes with the full-row leading dimension
      mine = st.buffer("g", B * ld)
      mine.view(B, ld)[:, :grad.shape[1] * F].copy_(grad.view(B, -1))
      st.sb.barrier()
      ptrs = st.sb.ptrs_for(mine)
      out = torch.empty(B, len(held) * Tc, F, dtype=grad.dtype, device=grad.device)
      tmp = torch.empty(B, Tc * F, dtype=grad.dtype, device=grad.device)
      for slot, c in enumerate(held):
        acc = grad[:, c * Tc:(c + 1) * Tc].reshape(B, -1).float()
        for r in layout.users(c):
          if r == rank:
            continue
          st.sb.peer_copy_2d(ptrs[r] + 2 * c * Tc * F, tmp, B, Tc * F, ld)
          acc += tmp
        out[:, slot * Tc:(slot + 1) * Tc] = acc.view(B, Tc, F).to(grad.dtype)
      return out, None, None
    full = torch.zeros(B, n_all * Tc, F, dtype=grad.dtype, device=grad.device)
    full[:, :grad.shape[1]] = grad
    dist.all_reduce(full, group=group)
    return torch.cat([full[:, c * Tc:(c + 1) * Tc] for c in held], dim=1), None, None


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, group, layout: Layout, attend) -> torch.Tensor:
  """Causal attention of this rank's query chunks over the global key prefix of each. q [B, T, N, H],
  k / v [B, T, K, H] local; `attend(q, k, v)` is rectangular causal attention with the queries aligned to the
  end of the keys. K and V travel together (one transfer, one barrier per call)."""
  rank = dist.get_rank(group)
  held = layout.chunks(rank)
  B, T, K, H = k.shape
  Tc = T // len(held)
  kv = _PrefixGather.apply(torch.stack((k, v), dim=2).reshape(B, T, 2 * K * H), group, layout)
  kv = kv.view(B, -1, 2, K, H)
  outs = []
  for slot, c in enumerate(held):
    n = (c + 1) * Tc
    kc, vc = kv[:, :n, 0], kv[:, :n, 1]
    if n < kv.shape[1] and B > 1:      # a shorter prefix of a batch is not one strided row range: copy it out
      kc, vc = kc.contiguous(), vc.contiguous()
    outs.append(attend(q[:, slot * Tc:(slot + 1) * Tc], kc, vc))
  return outs[0] if len(outs) == 1 else torch.cat(outs, dim=1)


def causal_prefix(k: torch.Tensor, v: torch.Tensor, group, T: int):
  """Keys / values [0, (rank + 1) T) of the contiguous layout (kept for callers that run attention themselves)."""
  layout = Layout(dist.get_world_size(group), "contiguous")
  B, _, K, H = k.shape
  kv = _PrefixGather.apply(torch.stack((k, v), dim=2).reshape(B, T, 2 * K * H), group, layout).view(B, -1, 2, K, H)
  return kv[:, :, 0], kv[:, :, 1]


# ------------------------------------------------------------------ model wiring
def shard_model_sp(model: torch.nn.Module, mesh, axis: str = "sp", layout: str = "contiguous") -> torch.nn.Module:
  from ..models.transformer import Attention
  group = mesh.group(axis)
  if mesh.axis_size(axis) == 1:
    return model
  lay = Layout(mesh.axis_size(axis), layout)
  for mod in model.modules():
    if isinstance(mod, Attention):
      mod.sp_group, mod.sp_layout = group, lay
  model.sp_group, model.sp_layout = group, lay
  return model


def _rank_slices(L: int, layout: Layout, rank: int) -> List[slice]:
  if L % layout.num_chunks:
    raise ValueError(f"sequence length {L} does not divide into {layout.num_chunks} chunks "
                     f"({layout.kind} layout over {layout.world} sequence-parallel ranks)")
  Tc = L // layout.num_chunks
  return [slice(c * Tc, (c + 1) * Tc) for c in layout.chunks(rank)]


def local_chunk(tokens: torch.Tensor, mesh, axis: str = "sp", layout: str = "contiguous"):
  """This rank's part of [B, L] tokens and the global positions that go with it."""
  lay = Layout(mesh.axis_size(axis), layout)
  parts = _rank_slices(tokens.shape[1], lay, mesh.axis_index(axis))
  pos = torch.cat([torch.arange(s.start, s.stop, device=tokens.device) for s in parts])
  return torch.cat([tokens[:, s] for s in parts], dim=1), pos[None].expand(tokens.shape[0], -1)


def local_rows(x: torch.Tensor, mesh, axis: str = "sp", layout: str = "contiguous", dim: int = 1) -> torch.Tensor:
  """The slice of any per-token tensor (targets, masks, reference logits) that matches `local_chunk`."""
  lay = Layout(mesh.axis_size(axis), layout)
  parts = _rank_slices(x.shape[dim], lay, mesh.axis_index(axis))
  return torch.cat([x.narrow(dim, s.start, s.stop - s.start) for s in parts], dim=dim)


def reduce_gradients(model: torch.nn.Module, group) -> None:
  """Sums parameter gradients over the sequence shards (models without a flat store)."""
  for p in model.parameters():
    if p.grad is not None:
      dist.all_reduce(p.grad, group=group)
