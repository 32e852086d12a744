"""Expert parallelism for `models.transformer.MoELayer`.

Experts are split evenly over the ranks of one mesh axis; every rank routes its own tokens,
sends each (token, expert) row to the rank that owns the expert, runs its local experts over
what it received (rows grouped by expert, one grouped MLP), and sends the results back, where
they are weighted and summed per token - the dispatch / grouped-GEMM / combine structure of
tunix/models/qwen3/model.py:837-1042.

The exchange is `all_to_all_single` with per-rank row counts (NCCL); it is differentiable (the
gradient of an all-to-all is the all-to-all with the counts swapped). On backends without
all-to-all (gloo in the CPU tests) rows travel through a padded all-gather instead.
"""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist


def _exchange(rows: torch.Tensor, send: List[int], recv: List[int], group) -> torch.Tensor:
  """rows [sum(send), D] ordered by destination rank -> [sum(recv), D] ordered by source rank."""
  world = dist.get_world_size(group)
  out = rows.new_empty((sum(recv),) + tuple(rows.shape[1:]))
  if dist.get_backend(group) != "gloo":
    dist.all_to_all_single(out, rows.contiguous(), output_split_sizes=recv, input_split_sizes=send, group=group)
    return out
  # gloo: everybody publishes its padded send buffer and its split table
  me = dist.get_rank(group)
  table = torch.tensor(send, dtype=torch.int64)
  tables = [torch.empty_like(table) for _ in range(world)]
  dist.all_gather(tables, table, group=group)
  most = max(int(t.sum()) for t in tables)
  pad = rows.new_zeros((most,) + tuple(rows.shape[1:]))
  pad[:rows.shape[0]] = rows
  bufs = [torch.empty_like(pad) for _ in range(world)]
  dist.all_gather(bufs, pad, group=group)
  pos = 0
  for src in range(world):
    start = int(tables[src][:me].sum())
    n = int(tables[src][me])
    out[pos:pos + n] = bufs[src][start:start + n]
    pos += n
  return out


class _AllToAllRows(torch.autograd.Function):

  @staticmethod
  def forward(ctx, rows, send, recv, group):
    ctx.send, ctx.recv, ctx.group = send, recv, group
    return _exchange(rows, send, recv, group)

  @staticmethod
  def backward(ctx, grad):
    return _exchange(grad.contiguous(), ctx.recv, ctx.send, ctx.group), None, None, None


def shard_experts(model: torch.nn.Module, mesh, axis: str = "fsdp") -> torch.nn.Module:
  """Keeps only this rank's slice of every MoE layer's stacked expert weights and marks the layer
  for expert-parallel execution. Call on identically initialised replicas."""
  from ..models.transformer import MoELayer
  group = mesh.group(axis)
  ep, r = mesh.axis_size(axis), mesh.axis_index(axis)
  for mod in model.modules():
    if isinstance(mod, MoELayer):
      E = mod.cfg.num_experts
      if E % ep:
        raise ValueError(f"{E} experts do not divide over {ep} ranks")
      per = E // ep
      with torch.no_grad():
        mod.gate_up_proj.data = mod.gate_up_proj.data[r * per:(r + 1) * per].clone()
        mod.down_proj.data = mod.down_proj.data[r * per:(r + 1) * per].clone()
      mod.ep_group, mod.ep_size, mod.ep_rank = group, ep, r
      mod.gate_up_proj.is_expert_parallel = True      # gradients of expert weights are not reduced over `axis`
      mod.down_proj.is_expert_parallel = True
  return model


def ep_forward(layer, x2: torch.Tensor, topv: torch.Tensor, topi: torch.Tensor) -> torch.Tensor:
  """x2 [T, D] local tokens, topv/topi [T, k] routing weights and expert ids -> [T, D]."""
  cfg = layer.cfg
  group, ep = layer.ep_group, layer.ep_size
  E, k = cfg.num_experts, cfg.num_experts_per_tok
  per = E // ep
  flat_e = topi.reshape(-1)
  order = torch.argsort(flat_e, stable=True)           # by expert, hence by destination rank
  tok = order // k
  xs = x2.index_select(0, tok)
  counts = torch.bincount(flat_e, minlength=E)          # rows per global expert, this rank's tokens
  # every rank learns how many rows it gets from whom, per local expert
  counts_in = torch.empty_like(counts)
  if dist.get_backend(group) != "gloo":
    dist.all_to_all_single(counts_in, counts, group=group)
  else:
    allc = [torch.empty_like(counts) for _ in range(ep)]
    dist.all_gather(allc, counts, group=group)
    me = dist.get_rank(group)
    counts_in = torch.cat([c[me * per:(me + 1) * per] for c in allc])
  send = counts.view(ep, per).sum(1).tolist()
  recv_table = counts_in.view(ep, per)                  # [source rank, local expert]
  recv = recv_table.sum(1).tolist()
  got = _AllToAllRows.apply(xs, send, recv, group)
  # received rows are ordered (source, expert); the grouped MLP wants (expert, source)
  src_exp = recv_table.reshape(-1)
  seg_expert = torch.arange(per, device=got.device).repeat(ep)
  row_expert = torch.repeat_interleave(seg_expert, src_exp)
  perm = torch.argsort(row_expert, stable=True)
  local_counts = recv_table.sum(0).tolist()
  ys = layer.experts(got.index_select(0, perm), local_counts, 0)
  back = ys.new_zeros(ys.shape).index_add(0, perm, ys)      # undo the regrouping (differentiable scatter)
  ret = _AllToAllRows.apply(back, recv, send, group)
  w = topv.reshape(-1).index_select(0, order).to(ret.dtype)
  return torch.zeros_like(x2).index_add_(0, tok, ret * w[:, None])
