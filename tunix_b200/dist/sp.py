"""Sequence parallelism: activations sharded along the sequence over one mesh axis, attention with
all-gathered keys / values (the reference's `'sp'` axis keeps K/V whole per shard and shards only the
queries; it has no ring or Ulysses variant - tunix/models/qwen3/model.py:576-672, tunix/sft/sharding_utils.py).

`shard_model_sp(model, mesh, axis)` marks every attention block. Rank r of the axis then feeds the model
tokens [r T, (r + 1) T) of each row together with their GLOBAL positions; everything outside attention is
per token and needs no communication. Inside attention the local K/V chunk is all-gathered along the
sequence and, because attention is causal, rank r only uses keys [0, (r + 1) T): its queries are the last
T positions of that prefix, which is exactly the rectangular causal case the flash kernels implement
(queries aligned to the end of the keys). The gradient of the all-gather is a reduce-scatter, so dK / dV
contributions from later ranks flow back to the owners of the keys. Parameter gradients are partial sums
over the sequence shards and are reduced over the axis like data-parallel gradients.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


class _GatherSeq(torch.autograd.Function):
  """[B, T, ...] local chunk -> [B, world * T, ...]; backward: sum over ranks of the slice that is ours."""

  @staticmethod
  def forward(ctx, x, group):
    world = dist.get_world_size(group)
    ctx.group, ctx.world, ctx.rank = group, world, dist.get_rank(group)
    parts = [torch.empty_like(x) for _ in range(world)]
    dist.all_gather(parts, x.contiguous(), group=group)
    return torch.cat(parts, dim=1)

  @staticmethod
  def backward(ctx, grad):
    T = grad.shape[1] // ctx.world
    grad = grad.contiguous()
    if dist.get_backend(ctx.group) == "gloo":
      dist.all_reduce(grad, group=ctx.group)
      return grad[:, ctx.rank * T:(ctx.rank + 1) * T].contiguous(), None
    out = torch.empty_like(grad[:, :T])
    chunks = [grad[:, r * T:(r + 1) * T].contiguous() for r in range(ctx.world)]
    dist.reduce_scatter(out, chunks, group=ctx.group)
    return out, None


def gather_sequence(x: torch.Tensor, group) -> torch.Tensor:
  return _GatherSeq.apply(x, group)


def causal_prefix(k: torch.Tensor, v: torch.Tensor, group, T: int):
  """All-gathered K/V cut to the keys a rank's queries may see: [0, (rank + 1) T)."""
  r = dist.get_rank(group)
  kg, vg = gather_sequence(k, group), gather_sequence(v, group)
  return kg[:, :(r + 1) * T], vg[:, :(r + 1) * T]


def shard_model_sp(model: torch.nn.Module, mesh, axis: str = "sp") -> torch.nn.Module:
  from ..models.transformer import Attention
  group = mesh.group(axis)
  if mesh.axis_size(axis) == 1:
    return model
  for mod in model.modules():
    if isinstance(mod, Attention):
      mod.sp_group = group
  model.sp_group = group
  return model


def local_chunk(tokens: torch.Tensor, mesh, axis: str = "sp"):
  """This rank's slice of [B, L] tokens and the global positions that go with it."""
  w, r = mesh.axis_size(axis), mesh.axis_index(axis)
  L = tokens.shape[1]
  if L % w:
    raise ValueError(f"sequence length {L} does not divide over {w} sequence-parallel ranks")
  T = L // w
  pos = torch.arange(r * T, (r + 1) * T, device=tokens.device)[None].expand(tokens.shape[0], T)
  return tokens[:, r * T:(r + 1) * T], pos


def reduce_gradients(model: torch.nn.Module, group) -> None:
  """Sums parameter gradients over the sequence shards (models without a flat store)."""
  for p in model.parameters():
    if p.grad is not None:
      dist.all_reduce(p.grad, group=group)
