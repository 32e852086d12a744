"""Expert parallelism for `models.transformer.MoELayer`.

Experts are split evenly over the ranks of one mesh axis; every rank routes its own tokens,
sends each (token, expert) row to the rank that owns the expert, runs its local experts over
what it received (rows grouped by expert, one grouped MLP), and sends the results back, where
they are weighted and summed per token - the dispatch / grouped-GEMM / combine structure of
tunix/models/qwen3/model.py:837-1042.

On CUDA the exchange is done by our own kernels over NVLink peer memory (`ep_forward_peer`, below):
rows are stored straight into the owner's expert-major buffer and results are pulled back, with the
placement computed on the device. The portable path is `all_to_all_single` with per-rank row counts;
it is differentiable (the gradient of an all-to-all is the all-to-all with the counts swapped). On
backends without all-to-all (gloo in the CPU tests) rows travel through a padded all-gather instead.
"""
from __future__ import annotations

import dataclasses
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
  if peer_supported(layer, x2):
    return ep_forward_peer(layer, x2, topv, topi)
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


# ------------------------------------------------------------------------------ peer-memory path
# Dispatch and combine as our own kernels over NVLink peer memory (`csrc/moe_dispatch.cu`): rows
# are stored straight into the owning rank's expert-major padded buffer and results are pulled
# back, weighted and summed in one pass. Everything that decides the placement stays on the
# device: the only collective is an all-gather of the [E] routing histogram.

@dataclasses.dataclass
class PeerPlan:
  """Placement of this rank's routed rows on the owning ranks, and this rank's receive layout."""
  dest_rank: torch.Tensor      # [n] int32
  dest_row: torch.Tensor       # [n] int32: row in the destination's [capacity, D] buffer
  layout: "moe_ops.PaddedLayout"   # receive side: offsets / tile_expert of the local experts
  valid: torch.Tensor          # [capacity] bool: rows that hold a routed row (padding rows are False)


def peer_plan(flat_e: torch.Tensor, table: torch.Tensor, me: int, capacity: int) -> PeerPlan:
  """flat_e [n]: global expert of every routed row of this rank; table [ep, E]: rows per (source rank,
  expert). Each expert's block on its owner is ordered by source rank and padded to 128 rows. Pure tensor
  code, the same on every backend."""
  from ..ops import moe as moe_ops
  ep, E = table.shape
  per = E // ep
  T = moe_ops.TILE
  ids = flat_e.reshape(-1).long()
  table = table.long()
  tot = table.sum(0)
  padded = (tot + (T - 1)) // T * T
  pv = padded.view(ep, per)
  start = (torch.cumsum(pv, 1) - pv).reshape(E)           # first row of expert e on its owner
  before = (torch.cumsum(table, 0) - table)[me]            # rows of lower source ranks, per expert
  n = ids.numel()
  order = torch.argsort(ids, stable=True)
  mine = table[me]
  first = torch.cumsum(mine, 0) - mine
  rank_sorted = torch.arange(n, device=ids.device) - first[ids[order]]
  rank_in = torch.empty_like(rank_sorted).index_copy_(0, order, rank_sorted)
  dest_row = start[ids] + before[ids] + rank_in
  dest_rank = ids // per
  # receive side
  offsets = torch.zeros(per + 1, dtype=torch.long, device=ids.device)
  offsets[1:] = torch.cumsum(pv[me], 0)
  tile_start = torch.arange(capacity // T, device=ids.device) * T
  te = torch.searchsorted(offsets[1:].contiguous(), tile_start, right=True)
  te = torch.where(tile_start < offsets[per], te, torch.full_like(te, -1))
  rows = torch.arange(capacity, device=ids.device)
  e_of_row = te.repeat_interleave(T).clamp(min=0)
  valid = (te.repeat_interleave(T) >= 0) & (rows < offsets[e_of_row] + tot.view(ep, per)[me][e_of_row])
  lay = moe_ops.PaddedLayout(capacity, dest_row, offsets.int(), te.int(), per)
  return PeerPlan(dest_rank.int(), dest_row.int(), lay, valid)


class PeerWorkspace:
  """Two symmetric [capacity, D] bf16 buffers per rank: `recv` is written by the peers (dispatch, and the
  scaled output gradients on the way back), `send` is read by the peers (expert outputs, and input
  gradients on the way back). A write into either is always separated from its previous readers by a
  device-side barrier that every reader reaches after reading."""

  def __init__(self, group, device: torch.device, capacity: int, D: int):
    from . import symm
    self.sb = symm.SymmetricBuffers(group, device)
    self.capacity, self.D = capacity, D
    self.recv = self.sb.alloc("moe_recv", capacity * D, torch.bfloat16).view(capacity, D)
    self.send = self.sb.alloc("moe_send", capacity * D, torch.bfloat16).view(capacity, D)
    self.recv.zero_()
    self.send.zero_()
    self.sb.rendezvous()
    self.world, self.rank = self.sb.world, self.sb.rank
    self._recv_ptrs = symm._ptr_array(self.sb.peer_ptrs["moe_recv"])
    self._send_ptrs = symm._ptr_array(self.sb.peer_ptrs["moe_send"])

  def barrier(self):
    self.sb.barrier()

  def dispatch(self, src: torch.Tensor, k: int, scale: Optional[torch.Tensor], plan: PeerPlan) -> None:
    from ..ops import _lib
    n = plan.dest_row.numel()
    rc = _lib.require().tx_moe_dispatch_rows(
        src.data_ptr(), src.stride(0), None, k, scale.data_ptr() if scale is not None else None,
        plan.dest_rank.data_ptr(), plan.dest_row.data_ptr(), self._recv_ptrs, self.world, n, self.D, self.capacity,
        _lib.status_word(src.device).data_ptr(), _lib.stream_ptr())
    _lib.check_rc(rc, "tx_moe_dispatch_rows")

  def combine(self, weights: Optional[torch.Tensor], k: int, T: int, plan: PeerPlan, keep_rows: bool):
    from ..ops import _lib
    out = torch.empty((T, self.D), dtype=torch.bfloat16, device=self.recv.device)
    gathered = torch.empty((T * k, self.D), dtype=torch.bfloat16, device=out.device) if keep_rows else None
    rc = _lib.require().tx_moe_combine_rows(
        self._send_ptrs, self.world, plan.dest_rank.data_ptr(), plan.dest_row.data_ptr(),
        weights.data_ptr() if weights is not None else None, k, out.data_ptr(), out.stride(0),
        gathered.data_ptr() if gathered is not None else None, T, self.D, self.capacity,
        _lib.status_word(out.device).data_ptr(), _lib.stream_ptr())
    _lib.check_rc(rc, "tx_moe_combine_rows")
    return out, gathered


_WORKSPACES = {}


def peak_capacity_need() -> Optional[float]:
  """Largest (padded rows received) / (rows routed) any layer of this rank has seen: the capacity factor that would
  have sufficed. One device-to-host read; meant for the end of a run."""
  vals = [float(ws.peak_need) for ws in _WORKSPACES.values() if getattr(ws, "peak_need", None) is not None]
  return max(vals) if vals else None


def peer_workspace(group, device: torch.device, n_rows: int, D: int, ep: int, per: int,
                   capacity_factor: Optional[float]) -> PeerWorkspace:
  """The workspace of (group, D), grown when a larger step arrives. Collective when it (re)allocates, so
  every rank must see the same row count per step (pad the batch otherwise)."""
  from ..ops import moe as moe_ops
  worst = n_rows * ep
  want = worst if capacity_factor is None else min(worst, int(capacity_factor * n_rows) + 1)
  capacity = moe_ops.padded_rows(want, per)
  key = (id(group), D)
  ws = _WORKSPACES.get(key)
  if ws is None or ws.capacity < capacity:
    ws = PeerWorkspace(group, device, capacity, D)
    _WORKSPACES[key] = ws
  return ws


def _masked_copy(buf: torch.Tensor, valid: torch.Tensor) -> torch.Tensor:
  return torch.where(valid[:, None], buf, torch.zeros((), dtype=buf.dtype, device=buf.device))


class _PeerDispatch(torch.autograd.Function):

  @staticmethod
  def forward(ctx, x2, plan, ws, k):
    ws.dispatch(x2, k, None, plan)
    ws.barrier()                                   # every peer's rows have landed
    ctx.plan, ctx.ws, ctx.k, ctx.T = plan, ws, k, x2.shape[0]
    return _masked_copy(ws.recv, plan.valid)       # private copy with zero padding rows

  @staticmethod
  def backward(ctx, dx_rows):
    ws, plan = ctx.ws, ctx.plan
    ws.send.copy_(dx_rows)
    ws.barrier()
    dx, _ = ws.combine(None, ctx.k, ctx.T, plan, keep_rows=False)
    return dx, None, None, None


class _PeerCombine(torch.autograd.Function):

  @staticmethod
  def forward(ctx, y_rows, topv, plan, ws):
    T, k = topv.shape
    ws.send.copy_(y_rows)
    ws.barrier()                                   # every rank's expert outputs are in place
    w = topv.reshape(-1).float().contiguous()
    out, gathered = ws.combine(w, k, T, plan, keep_rows=True)
    ctx.save_for_backward(gathered, w)
    ctx.plan, ctx.ws, ctx.shape = plan, ws, (T, k)
    return out

  @staticmethod
  def backward(ctx, dout):
    gathered, w = ctx.saved_tensors
    ws, plan = ctx.ws, ctx.plan
    T, k = ctx.shape
    dout = dout.contiguous()
    dtopv = torch.einsum("tkd,td->tk", gathered.view(T, k, -1).float(), dout.float())
    ws.dispatch(dout, k, w, plan)                  # rows of w * dout go back to the experts' owners
    ws.barrier()
    return _masked_copy(ws.recv, plan.valid), dtopv, None, None


def peer_supported(layer, x2: torch.Tensor) -> bool:
  import os
  from ..ops import moe as moe_ops
  if os.environ.get("TUNIX_B200_EP_PEER", "1") == "0" or not x2.is_cuda:
    return False
  if dist.get_backend(layer.ep_group) != "nccl":
    return False
  return moe_ops.grouped_supported(x2, layer.gate_up_proj) and moe_ops.grouped_supported(x2, layer.down_proj)


def ep_forward_peer(layer, x2: torch.Tensor, topv: torch.Tensor, topi: torch.Tensor) -> torch.Tensor:
  """Expert-parallel routed MLP with peer-memory dispatch / combine and grouped tensor-core GEMMs."""
  from ..ops import moe as moe_ops
  cfg = layer.cfg
  group, ep = layer.ep_group, layer.ep_size
  E, k = cfg.num_experts, cfg.num_experts_per_tok
  per = E // ep
  T, D = x2.shape
  flat_e = topi.reshape(-1)
  counts = moe_ops.count_rows(flat_e, E)
  table = torch.empty((ep, E), dtype=counts.dtype, device=counts.device)
  dist.all_gather_into_tensor(table, counts, group=group)
  ws = peer_workspace(group, x2.device, T * k, D, ep, per, getattr(layer, "ep_capacity_factor", None))
  plan = peer_plan(flat_e, table, layer.ep_rank, ws.capacity)
  need = plan.layout.offsets[-1:].float() / float(T * k)       # padded rows this rank receives / rows it routes
  ws.peak_need = need if getattr(ws, "peak_need", None) is None else torch.maximum(ws.peak_need, need)
  x_rows = _PeerDispatch.apply(x2.contiguous(), plan, ws, k)
  y_rows = moe_ops.grouped_mlp_padded(x_rows, plan.layout, layer.gate_up_proj, layer.down_proj, cfg.activation)
  return _PeerCombine.apply(y_rows, topv, plan, ws)
