"""Fully sharded data parallel training sized for 180 GB GPUs.

Layout. All trainable parameters of a model live in one flat bf16 buffer, their fp32 gradient
accumulators (`param.main_grad`) in one flat fp32 buffer. The flat index space is cut into
`world` contiguous shards; rank r owns the fp32 master weights and both Adam moments of shard r
only (ZeRO-style sharding of everything that is touched once per optimizer step).

The bf16 compute copy stays gathered for the whole optimizer step: with 180 GB of HBM3e per GPU
a resident 8-70B bf16 replica costs less than re-gathering every layer for every micro-batch
and for every recomputation, and NVLink traffic per optimizer step drops to one reduce-scatter
of the gradients plus one all-gather of the updated parameters regardless of the number of
micro-batches. (The reference shards on the 'fsdp' mesh axis and lets the compiler insert a
gather before each consuming matmul, tunix/models/llama3/model.py:65-82.)

Optimizer step, once all micro-batches have accumulated into the local flat gradient:

  1. reduce-scatter: rank r sums shard r of every rank's gradient buffer,
  2. fp32 global norm of the summed gradient (sum of squares per shard + all-reduce),
  3. AdamW on shard r with scale = clip / sum(denominators), refreshing shard r of the bf16 copy,
  4. all-gather of the bf16 shards.

Two transports implement 1 and 3+4: `nccl` (library collectives: the baseline) and `p2p`
(`tunix_b200.dist.symm`: the gradient and parameter buffers are allocated in peer-mapped
symmetric memory, one kernel pulls and sums the peers' gradient shards over NVLink, another
applies AdamW and pushes the updated bf16 values straight into every peer's parameter buffer).
"""
from __future__ import annotations

import logging
import math
import os
from typing import Any, Dict, List, Mapping, Optional, Tuple

import torch
import torch.distributed as dist

from . import mesh as mesh_lib

log = logging.getLogger(__name__)

_ALIGN = 2048   # elements; keeps every shard boundary 16-byte aligned for any dtype and vector width


class FlatParamStore:
  """Flat bf16 parameters + flat fp32 gradients, sharded optimizer state."""

  def __init__(self, model: torch.nn.Module, mesh: Optional[mesh_lib.Mesh] = None, axis: str = "fsdp",
               transport: Optional[str] = None, only_trainable: bool = True):
    self.mesh = mesh
    self.axis = axis
    self.group = mesh.group(axis) if mesh is not None else None
    self.world = mesh.axis_size(axis) if mesh is not None else 1
    self.rank = mesh.axis_index(axis) if mesh is not None else 0
    every = [(n, p) for n, p in model.named_parameters() if p.requires_grad or not only_trainable]
    # expert-parallel parameters differ per rank: they get a rank-local region (no reduction, whole optimizer state)
    local = [(n, p) for n, p in every if getattr(p, "is_expert_parallel", False)]
    params = [(n, p) for n, p in every if not getattr(p, "is_expert_parallel", False)]
    if not params:
      raise ValueError("model has no trainable parameters")
    dev = params[0][1].device
    dtype = params[0][1].dtype
    if any(p.dtype != dtype or p.device != dev for _, p in params):
      raise ValueError("FlatParamStore needs all trainable parameters on one device with one dtype")
    self.device, self.dtype = dev, dtype
    self.names = [n for n, _ in params]
    self.shapes = {n: tuple(p.shape) for n, p in params}
    self.offsets: Dict[str, int] = {}
    off = 0
    for n, p in params:
      self.offsets[n] = off
      off += (p.numel() + 7) // 8 * 8     # 16-byte aligned starts (TMA / vector loads)
    unit = _ALIGN * self.world
    self.numel = (off + unit - 1) // unit * unit
    self.used = off
    self.shard_numel = self.numel // self.world
    self.transport = transport or os.environ.get("TUNIX_FSDP_TRANSPORT", "p2p" if self.world > 1 else "local")
    self.symm = None
    if self.world > 1 and self.transport == "p2p":
      from . import symm
      try:
        self.symm = symm.SymmetricBuffers(self.group, dev)
        self.flat_param = self.symm.alloc("fsdp_param", self.numel, dtype)
        self.flat_grad = self.symm.alloc("fsdp_grad", self.numel, torch.float32)
        self.symm.rendezvous()
      except Exception as e:
        log.warning("symmetric memory unavailable (%s); falling back to NCCL transport", e)
        self.symm = None
        self.transport = "nccl"
    if self.symm is None:
      self.flat_param = torch.zeros(self.numel, dtype=dtype, device=dev)
      self.flat_grad = torch.zeros(self.numel, dtype=torch.float32, device=dev)
    else:
      self.flat_param.zero_()
      self.flat_grad.zero_()
    with torch.no_grad():
      for n, p in params:
        o = self.offsets[n]
        view = self.flat_param[o:o + p.numel()].view(p.shape)
        view.copy_(p.data)
        p.data = view
        p.main_grad = self.flat_grad[o:o + p.numel()].view(p.shape)
    self.params = dict(params)
    self.local_names = [n for n, _ in local]
    self.local_shapes = {n: tuple(p.shape) for n, p in local}
    self.local_offsets: Dict[str, int] = {}
    off = 0
    for n, p in local:
      self.local_offsets[n] = off
      off += (p.numel() + 7) // 8 * 8
    self.local_numel = off
    self.local_param = self.local_grad = None
    if local:
      self.local_param = torch.zeros(off, dtype=dtype, device=dev)
      self.local_grad = torch.zeros(off, dtype=torch.float32, device=dev)
      with torch.no_grad():
        for n, p in local:
          o = self.local_offsets[n]
          view = self.local_param[o:o + p.numel()].view(p.shape)
          view.copy_(p.data)
          p.data = view
          p.main_grad = self.local_grad[o:o + p.numel()].view(p.shape)
      self.params.update(dict(local))
    lo = self.rank * self.shard_numel
    self.shard = slice(lo, lo + self.shard_numel)
    self._scratch: Dict[str, torch.Tensor] = {}
    self.grad_shard: Optional[torch.Tensor] = None   # fp32 [shard_numel]: reduced gradient of my shard
    if self.world > 1:
      self.grad_shard = torch.zeros(self.shard_numel, dtype=torch.float32, device=dev)

  # ---- optimizer state ------------------------------------------------------------------
  def init_state(self, tx) -> Dict[str, Any]:
    """Flat fp32 master / mu / nu for this rank's shard (names follow the optax tree)."""
    master = self.flat_param[self.shard].float()
    st: Dict[str, Any] = {
        "count": torch.zeros((), dtype=torch.int32),
        "master": {"flat": master},
        "mu": {"flat": torch.zeros_like(master)},
        "nu": {"flat": torch.zeros_like(master)},
    }
    if self.local_param is not None:
      lm = self.local_param.float()
      st["master"]["local"], st["mu"]["local"], st["nu"]["local"] = lm, torch.zeros_like(lm), torch.zeros_like(lm)
    if getattr(tx, "exposes_hyperparams", False):
      from .. import optim
      st["hyperparams"] = {"learning_rate": torch.tensor(optim._lr_at(tx._lr, 0), dtype=torch.float32)}
    return st

  def _buf(self, name: str, n: int = 1) -> torch.Tensor:
    t = self._scratch.get(name)
    if t is None:
      t = torch.zeros(n, dtype=torch.float32, device=self.device)
      self._scratch[name] = t
    return t

  # ---- the optimizer step ------------------------------------------------------------------
  @torch.no_grad()
  def step(self, tx, state: Dict[str, Any], denom: torch.Tensor, max_grad_norm: Optional[float]) -> torch.Tensor:
    """Reduces gradients and denominators over the data-parallel group, applies the fused AdamW
    update to this rank's shard and republishes the bf16 parameters. Returns the fp32 global
    gradient norm (device scalar). `denom` is this rank's summed loss denominator."""
    from ..ops import kernels
    d = self._buf("denom")
    d.copy_(denom.reshape(1))
    ss = self._buf("sumsq")
    if self.world == 1:
      g = self.flat_grad
    elif self.symm is not None:
      self.symm.reduce_scatter_sum(self.flat_grad, self.grad_shard, self.rank)
      g = self.grad_shard
    elif self.device.type == "cuda":
      dist.reduce_scatter_tensor(self.grad_shard, self.flat_grad, op=dist.ReduceOp.SUM, group=self.group)
      g = self.grad_shard
    else:
      # gloo (CPU ranks in tests) has no reduce-scatter: all-reduce and keep this rank's slice
      dist.all_reduce(self.flat_grad, op=dist.ReduceOp.SUM, group=self.group)
      self.grad_shard.copy_(self.flat_grad[self.shard])
      g = self.grad_shard
    if self.device.type == "cuda":
      kernels.sumsq(g, ss, accumulate=False)
    else:
      ss.copy_(g.double().pow(2).sum().float().reshape(1))
    if self.local_grad is not None:
      # every rank's expert gradients are distinct, so their squares simply join the sum over ranks
      if self.device.type == "cuda":
        kernels.sumsq(self.local_grad, ss, accumulate=True)
      else:
        ss.add_(self.local_grad.double().pow(2).sum().float())
    if self.world > 1:
      pack = self._buf("pack", 2)
      pack[0:1].copy_(ss)
      pack[1:2].copy_(d)
      dist.all_reduce(pack, op=dist.ReduceOp.SUM, group=self.group)
      ss.copy_(pack[0:1])
      d.copy_(pack[1:2])
    inv = self._buf("inv")
    torch.where(d == 0, torch.zeros_like(d), 1.0 / torch.where(d == 0, torch.ones_like(d), d), out=inv)
    norm, scale = self._buf("norm"), self._buf("scale")
    if self.device.type == "cuda":
      kernels.clip_scale(ss, inv, max_grad_norm or 0.0, norm, scale)
    else:
      # norm of the mean gradient; scale = 1/denom, times max_norm/norm when clipping applies
      norm.copy_(ss.sqrt() * inv)
      scale.copy_(inv)
      if max_grad_norm and float(norm) > max_grad_norm:
        scale.mul_(max_grad_norm / (float(norm) + 1e-6))
    inner = getattr(tx, "inner", tx)
    if self.local_grad is not None:
      self._local_update(inner, state, scale)
    if self.world > 1 and self.symm is not None:
      self.symm.adamw_allgather(inner, state, g, self.flat_param, self.shard, scale)
    else:
      inner.fused_flat_step(state["master"]["flat"], state["mu"]["flat"], state["nu"]["flat"], g,
                            self.flat_param[self.shard], state, scale, zero_grad=False)
      if self.world > 1:
        dist.all_gather_into_tensor(self.flat_param, self.flat_param[self.shard], group=self.group)
    self.flat_grad.zero_()
    return norm[0].clone()

  def _local_update(self, inner, state, scale: torch.Tensor) -> None:
    """AdamW over the rank-local (expert-parallel) region; same step count and schedule as the sharded part,
    whose update follows and advances the count."""
    from .. import optim
    from ..ops import kernels
    count = int(state["count"]) + 1
    kernels.adamw_step(state["master"]["local"], state["mu"]["local"], state["nu"]["local"], self.local_grad,
                       self.local_param, lr=optim._lr_at(inner._lr, count - 1), beta1=inner.b1, beta2=inner.b2,
                       eps=inner.eps, weight_decay=inner.weight_decay, step=count, grad_scale=scale, zero_grad=True)

  # ---- checkpoint support ---------------------------------------------------------------------
  def state_shards(self, state: Mapping[str, Any]) -> Dict[Tuple, Any]:
    """This rank's part of the optimizer state as a checkpoint tree whose sharded leaves are chunks of
    flat arrays: `mu/nu/master.flat` of shape [numel] cut into `world` chunks of [shard_numel] (rank r
    holds chunk r) and, with expert parallelism, `*.local` of shape [world * local_numel]. Every rank
    writes its own chunk files; nothing crosses the ranks."""
    from ..ckpt.orbax_layout import ShardedArray
    out: Dict[Tuple, Any] = {("count", "value"): torch.as_tensor(state["count"])}
    for k in ("mu", "nu", "master"):
      out[(k, "flat", "value")] = ShardedArray(state[k]["flat"], (self.numel,), (self.shard_numel,), (self.rank,))
      if "local" in state[k]:
        out[(k, "local", "value")] = ShardedArray(state[k]["local"], (self.world * self.local_numel,),
                                                  (self.local_numel,), (self.rank,))
    for n, v in (state.get("hyperparams") or {}).items():
      out[("hyperparams", n, "value")] = torch.as_tensor(v)
    return out

  def flat_index(self) -> Dict[str, Any]:
    """Where each parameter sits in the flat arrays of `state_shards` (JSON-serialisable)."""
    return {"format": "tunix_b200.flat_state.v1", "numel": self.numel, "used": self.used, "world": self.world,
            "shard_numel": self.shard_numel, "names": list(self.names),
            "offsets": [self.offsets[n] for n in self.names], "shapes": [list(self.shapes[n]) for n in self.names],
            "local_numel": self.local_numel, "local_names": list(self.local_names),
            "local_offsets": [self.local_offsets[n] for n in self.local_names],
            "local_shapes": [list(self.local_shapes[n]) for n in self.local_names]}

  @torch.no_grad()
  def load_state_shards(self, state: Dict[str, Any], index: Mapping[str, Any], read_rows) -> None:
    """Restores this rank's shard from flat arrays written by `state_shards`, possibly by a job of another
    size: `read_rows(name, lo, hi)` returns elements [lo, hi) of the stored 1-D array `name`. Parameter
    offsets do not depend on the number of ranks, so a rank's flat range is the same range of the file."""
    if list(index["names"]) != list(self.names) or list(index["offsets"]) != [self.offsets[n] for n in self.names]:
      raise ValueError("checkpointed optimizer state was written for a different parameter layout")
    lo, hi = self.shard.start, self.shard.stop
    for k in ("mu", "nu", "master"):
      part = read_rows(f"{k}.flat", lo, hi)
      state[k]["flat"].copy_(part.to(self.device, torch.float32))
      if "local" in state[k]:
        if index.get("world") != self.world or index.get("local_numel") != self.local_numel:
          raise ValueError("expert-parallel optimizer state can only be restored at the expert-parallel size "
                           f"it was saved with ({index.get('world')} ranks)")
        a = self.rank * self.local_numel
        state[k]["local"].copy_(read_rows(f"{k}.local", a, a + self.local_numel).to(self.device, torch.float32))

  def full_state_tensor(self, shard_tensor: torch.Tensor) -> torch.Tensor:
    """All-gathers a sharded state tensor (per-parameter views for export; checkpoints do not use this)."""
    if self.world == 1:
      return shard_tensor
    full = torch.empty(self.numel, dtype=shard_tensor.dtype, device=shard_tensor.device)
    dist.all_gather_into_tensor(full, shard_tensor.contiguous(), group=self.group)
    return full

  def unflatten(self, flat: torch.Tensor) -> Dict[str, torch.Tensor]:
    out = {}
    for n in self.names:
      o = self.offsets[n]
      numel = int(math.prod(self.shapes[n])) if self.shapes[n] else 1
      out[n] = flat[o:o + numel].view(self.shapes[n])
    return out

  def opt_state_tree(self, state: Mapping[str, Any]) -> Dict[str, Any]:
    """Per-parameter view of the sharded optimizer state (gathers the shards)."""
    out: Dict[str, Any] = {"count": state["count"]}
    for k in ("mu", "nu", "master"):
      out[k] = self.unflatten(self.full_state_tensor(state[k]["flat"]))
      if "local" in state[k]:          # this rank's experts only
        for n in self.local_names:
          o = self.local_offsets[n]
          out[k][n] = state[k]["local"][o:o + int(math.prod(self.local_shapes[n]))].view(self.local_shapes[n])
    if "hyperparams" in state:
      out["hyperparams"] = state["hyperparams"]
    return out

  @torch.no_grad()
  def load_opt_state_tree(self, state: Dict[str, Any], tree: Mapping[str, Any]) -> None:
    for k in ("mu", "nu", "master"):
      if k not in tree:
        continue
      full = torch.zeros(self.numel, dtype=torch.float32, device=self.device)
      for n, t in tree[k].items():
        if n in self.offsets:
          o = self.offsets[n]
          full[o:o + t.numel()].copy_(t.reshape(-1).to(self.device, torch.float32))
      state[k]["flat"].copy_(full[self.shard])
      if "local" in state[k]:
        for n, t in tree[k].items():
          if n in self.local_offsets:
            o = self.local_offsets[n]
            state[k]["local"][o:o + t.numel()].copy_(t.reshape(-1).to(self.device, torch.float32))
    if "count" in tree:
      state["count"] = torch.as_tensor(tree["count"]).to(torch.int32).reshape(())

  @torch.no_grad()
  def refresh_master_from_params(self, state: Dict[str, Any]) -> None:
    """After parameters were loaded into the bf16 buffer (checkpoint restore, weight import)."""
    state["master"]["flat"].copy_(self.flat_param[self.shard].float())
    if "local" in state["master"]:
      state["master"]["local"].copy_(self.local_param.float())


def shard_model(model: torch.nn.Module, mesh: Optional[mesh_lib.Mesh] = None, axis: str = "fsdp",
                transport: Optional[str] = None) -> torch.nn.Module:
  """Moves the trainable parameters of `model` into a `FlatParamStore` (attached as
  `model.flat_store`). With `mesh=None` the store is single-rank: same flat layout, fused
  one-kernel optimizer step, no communication. All ranks must start from identical weights
  (same seed) or call `broadcast_params` afterwards."""
  store = FlatParamStore(model, mesh, axis, transport)
  model.flat_store = store
  return model


def broadcast_params(model: torch.nn.Module, src: int = 0) -> None:
  store: FlatParamStore = model.flat_store
  if store.world > 1:
    ranks = store.mesh.ranks()
    dist.broadcast(store.flat_param, src=ranks[src], group=store.mesh.all_group())


class GradSync:
  """Marker handed to `PeftTrainer.with_grad_sync`; the reduction itself happens inside
  `FlatParamStore.step`. For models without a flat store it all-reduces the per-parameter
  accumulators (plain data parallelism)."""

  def __init__(self, model: torch.nn.Module, mesh: Optional[mesh_lib.Mesh], axis: str = "fsdp"):
    self.flat = getattr(model, "flat_store", None)
    self.group = mesh.group(axis) if mesh is not None else None
    self.world = mesh.axis_size(axis) if mesh is not None else 1

  def reduce(self, acc) -> None:
    if self.flat is not None or self.world == 1:
      return
    for g in acc.acc.values():
      dist.all_reduce(g, group=self.group)
    dist.all_reduce(acc.denom, group=self.group)

  def reduce_scalars(self, values):
    """Sum of host floats over the data-parallel group (metrics path)."""
    if self.world == 1:
      return list(values)
    dev = self.flat.device if self.flat is not None else ("cuda" if torch.cuda.is_available() else "cpu")
    t = torch.tensor(list(values), dtype=torch.float64, device=dev)
    dist.all_reduce(t, group=self.group)
    return t.tolist()

  def reduce_norm_sq(self, sq: torch.Tensor) -> torch.Tensor:
    return sq    # gradients are already identical on every rank after `reduce`
