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

Ownership is interleaved by bucket. The flat index space is cut into buckets of a few decoder layers
each (embedding first, head last, in parameter order); rank r owns the r-th slice of EVERY bucket, so the
reduce-scatter of a bucket can start as soon as the last micro-batch's backward has passed its layers -
it then runs on a side stream, hidden behind the rest of the backward pass - and all ranks' links carry
an equal share of every transfer. Only the bucket that finishes last (the embedding) is reduced after
the backward pass.

Two transports implement 1 and 3+4: `nccl` (library collectives: the baseline) and `p2p`
(`tunix_b200.dist.symm`: the gradient and parameter buffers are allocated in peer-mapped
symmetric memory, one kernel pulls and sums the peers' gradient shards over NVLink, another
applies AdamW and pushes the updated bf16 values straight into every peer's parameter buffer).
"""
from __future__ import annotations

import contextlib
import logging
import math
import os
from typing import Any, Dict, List, Mapping, Optional, Tuple

import torch
import torch.distributed as dist

from . import mesh as mesh_lib

log = logging.getLogger(__name__)

_ALIGN = 2048   # elements; keeps every shard boundary 16-byte aligned for any dtype and vector width
_BACKGROUND_CTAS = int(os.environ.get("TUNIX_FSDP_BACKGROUND_CTAS", "0"))    # 0: the full-grid kernel (measured best); n > 0: n long-lived CTAs
_BUCKET_ALIGN = _ALIGN * 16   # bucket boundaries: divisible into 16-byte aligned pieces for up to 16 ranks


def _layer_index(name: str) -> Optional[int]:
  parts = name.split(".")
  for a, b in zip(parts, parts[1:]):
    if a == "layers" and b.isdigit():
      return int(b)
  return None


def _bucket_id(name: str, layers_per_bucket: int) -> int:
  """Bucket order follows parameter order: what precedes the layers, groups of layers, what follows them."""
  li = _layer_index(name)
  if li is not None:
    return 1 + li // layers_per_bucket
  return 0 if name.startswith("embedder") else 1 << 30


class FlatParamStore:
  """Flat bf16 parameters + flat fp32 gradients, sharded optimizer state."""

  resident = True          # the whole bf16 model stays on every rank (`fsdp_sharded.ShardedParamStore`: False)

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
    # buckets: consecutive parameters grouped by decoder layer; a bucket starts on a boundary that does not
    # depend on the number of ranks, so a checkpoint's flat offsets are valid for any power-of-two job size
    per_bucket = self._layers_per_bucket()
    pow2 = self.world & (self.world - 1) == 0 and self.world <= 16
    ids = [_bucket_id(n, per_bucket) for n, _ in params] if (pow2 and per_bucket > 0) else None
    if ids is not None and any(b < a for a, b in zip(ids, ids[1:])):
      ids = None                       # parameter order does not follow the layer order: one bucket
    off, starts, prev = 0, [0], (ids[0] if ids else 0)
    for i, (n, p) in enumerate(params):
      if ids is not None and ids[i] != prev:
        off = (off + _BUCKET_ALIGN - 1) // _BUCKET_ALIGN * _BUCKET_ALIGN
        starts.append(off)
        prev = ids[i]
      self.offsets[n] = off
      off += (p.numel() + 7) // 8 * 8     # 16-byte aligned starts (TMA / vector loads)
    self.used = off
    unit = _BUCKET_ALIGN if ids is not None else _ALIGN * self.world
    self.numel = (off + unit - 1) // unit * unit
    bounds = starts + [self.numel]
    # this rank's pieces: (flat start, length, offset inside the rank's shard tensors), one per bucket
    self.buckets: List[Tuple[int, int]] = [(lo, hi - lo) for lo, hi in zip(bounds[:-1], bounds[1:])]
    self.pieces: List[Tuple[int, int, int]] = []
    so = 0
    for lo, n in self.buckets:
      per = n // self.world
      self.pieces.append((lo + self.rank * per, per, so))
      so += per
    self.shard_numel = so
    self._bucket_ids = ids
    self._allocate(model, params, local, transport)

  def _layers_per_bucket(self) -> int:
    return int(os.environ.get("TUNIX_FSDP_BUCKET_LAYERS", "4"))

  def _allocate(self, model: torch.nn.Module, params, local, transport: Optional[str]) -> None:
    """Resident layout: whole flat bf16 parameter and fp32 gradient buffers on every rank."""
    dev, dtype, ids = self.device, self.dtype, self._bucket_ids
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
    self._scratch: Dict[str, torch.Tensor] = {}
    self._reduced: set = set()             # buckets whose reduce-scatter already ran (overlapped with backward)
    self._armed = False
    self._layers_done = 0
    self._side = None
    self._bucket_of_layer: Dict[int, int] = {}
    self._layers_in_bucket: Dict[int, int] = {}
    if ids is not None:
      b = -1
      last = None
      for i, (n, _) in enumerate(params):
        if ids[i] != last:
          b += 1
          last = ids[i]
        li = _layer_index(n)
        if li is not None and li not in self._bucket_of_layer:
          self._bucket_of_layer[li] = b
          self._layers_in_bucket[b] = self._layers_in_bucket.get(b, 0) + 1
      self._install_backward_hooks(model)
    self.grad_shard: Optional[torch.Tensor] = None   # fp32 [shard_numel]: reduced gradient of my shard
    if self.world > 1:
      self.grad_shard = torch.zeros(self.shard_numel, dtype=torch.float32, device=dev)

  # ---- optimizer state ------------------------------------------------------------------
  def init_state(self, tx) -> Dict[str, Any]:
    """Flat fp32 master / mu / nu for this rank's shard (names follow the optax tree)."""
    master = self._my_part(self.flat_param).float()
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

  def _my_part(self, flat: torch.Tensor) -> torch.Tensor:
    """This rank's pieces of a flat [numel] tensor, concatenated in bucket order ([shard_numel])."""
    if len(self.pieces) == 1:
      lo, n, _ = self.pieces[0]
      return flat[lo:lo + n]
    return torch.cat([flat[lo:lo + n] for lo, n, _ in self.pieces])

  def _put_my_part(self, flat: torch.Tensor, part: torch.Tensor) -> None:
    for lo, n, so in self.pieces:
      flat[lo:lo + n].copy_(part[so:so + n])

  # ---- overlap of the gradient reduce-scatter with the last backward pass ----------------------------
  def _install_backward_hooks(self, model: torch.nn.Module) -> None:
    """The fused decoder-layer node calls `grad_ready_hook` of its first norm weight when the layer's backward
    (all its weight gradients included) has been issued."""
    layers = getattr(model, "layers", None)
    if layers is None or self.symm is None:
      return
    import functools
    for i, layer in enumerate(layers):
      w = getattr(getattr(layer, "input_layernorm", None), "w", None)
      if w is not None and i in self._bucket_of_layer:
        w.grad_ready_hook = functools.partial(self._layer_backward_done, i)

  def after_backward(self) -> None:
    """Called by the trainer when a backward pass has returned (the sharded-parameter store closes its last
    unit here)."""

  @contextlib.contextmanager
  def summon_full_params(self, writeback: bool = False):
    """Every parameter is whole inside the block: always true for this store."""
    yield self

  def arm_overlap(self) -> None:
    """Called by the trainer before the backward pass of the LAST micro-batch of an optimizer step: from now on
    a bucket whose layers have all run backward holds final gradients and may be reduced."""
    if self.symm is not None and self._bucket_of_layer:
      self._armed = True
      self._done_in_bucket: Dict[int, int] = {}

  def _layer_backward_done(self, layer: int) -> None:
    if not self._armed:
      return
    b = self._bucket_of_layer[layer]
    self._done_in_bucket[b] = self._done_in_bucket.get(b, 0) + 1
    if self._done_in_bucket[b] < self._layers_in_bucket[b]:
      return
    # every bucket after b in flat order (later layers, head) ran backward earlier: reduce all that are due
    due = [x for x in range(b, len(self.buckets)) if x not in self._reduced and
           all(self._done_in_bucket.get(y, 0) >= n for y, n in self._layers_in_bucket.items() if y >= x)]
    if not due:
      return
    from ..ops import _lib
    _lib.bind_thread()
    if self._side is None:
      self._side = torch.cuda.Stream(device=self.device, priority=-1)   # its few CTAs go first at kernel boundaries
    ev = torch.cuda.Event()
    ev.record(torch.cuda.current_stream(self.device))
    self._side.wait_event(ev)
    self.symm.barrier(channel=1, stream=self._side)        # every rank's gradients of these buckets are final
    for x in sorted(due):
      lo, n, so = self.pieces[x]
      self.symm.reduce_scatter_piece(self.flat_grad, self.grad_shard[so:so + n], lo, stream=self._side,
                                     background_ctas=_BACKGROUND_CTAS)
      self._reduced.add(x)

  # ---- the optimizer step ------------------------------------------------------------------
  def _norm_and_scale(self, g: torch.Tensor, ss: torch.Tensor, d: torch.Tensor, max_grad_norm: Optional[float]):
    """fp32 global norm of the summed gradient (`g`: this rank's reduced shard) and the factor the update
    multiplies it by: 1 / sum of denominators, times max_norm / norm when clipping applies. Both are
    device scalars; one small all-reduce carries the sum of squares and the denominator together."""
    from ..ops import kernels
    if self.device.type == "cuda":
      kernels.sumsq(g, ss, accumulate=False)
    else:
      ss.copy_(g.double().pow(2).sum().float().reshape(1))
    if getattr(self, "local_grad", None) is not None:
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
    return norm, scale

  @torch.no_grad()
  def step(self, tx, state: Dict[str, Any], denom: torch.Tensor, max_grad_norm: Optional[float]) -> torch.Tensor:
    """Reduces gradients and denominators over the data-parallel group, applies the fused AdamW
    update to this rank's shard and republishes the bf16 parameters. Returns the fp32 global
    gradient norm (device scalar). `denom` is this rank's summed loss denominator."""
    from ..ops import kernels
    d = self._buf("denom")
    d.copy_(denom.reshape(1))
    ss = self._buf("sumsq")
    self._armed = False
    if self.world == 1:
      g = self.flat_grad
    elif self.symm is not None:
      rest = [x for x in range(len(self.buckets)) if x not in self._reduced]
      if rest:
        self.symm.barrier()      # every rank's gradients are final before anybody reads them
        for x in rest:
          lo, n, so = self.pieces[x]
          self.symm.reduce_scatter_piece(self.flat_grad, self.grad_shard[so:so + n], lo)
      if self._side is not None and self._reduced:
        torch.cuda.current_stream(self.device).wait_stream(self._side)
      self._reduced = set()
      g = self.grad_shard
    elif self.device.type == "cuda":
      for (blo, bn), (_, n, so) in zip(self.buckets, self.pieces):
        dist.reduce_scatter_tensor(self.grad_shard[so:so + n], self.flat_grad[blo:blo + bn], op=dist.ReduceOp.SUM,
                                   group=self.group)
      g = self.grad_shard
    else:
      # gloo (CPU ranks in tests) has no reduce-scatter: all-reduce and keep this rank's pieces
      dist.all_reduce(self.flat_grad, op=dist.ReduceOp.SUM, group=self.group)
      self.grad_shard.copy_(self._my_part(self.flat_grad))
      g = self.grad_shard
    norm, scale = self._norm_and_scale(g, ss, d, max_grad_norm)
    inner = getattr(tx, "inner", tx)
    if self.local_grad is not None:
      self._local_update(inner, state, scale)
    if self.world > 1 and self.symm is not None:
      self.symm.adamw_allgather(inner, state, g, self.flat_param, self.pieces, scale)
    else:
      if self.world == 1:
        inner.fused_flat_step(state["master"]["flat"], state["mu"]["flat"], state["nu"]["flat"], g,
                              self.flat_param[:self.shard_numel], state, scale, zero_grad=False)
      else:
        mine = self._my_part(self.flat_param).contiguous()
        inner.fused_flat_step(state["master"]["flat"], state["mu"]["flat"], state["nu"]["flat"], g, mine, state, scale,
                              zero_grad=False)
        self._put_my_part(self.flat_param, mine)
        for (blo, bn), (lo, n, _) in zip(self.buckets, self.pieces):
          dist.all_gather_into_tensor(self.flat_param[blo:blo + bn], self.flat_param[lo:lo + n].clone(), group=self.group)
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
    rank-major arrays: `mu/nu/master.flat` of shape [world * shard_numel], chunk r = rank r's pieces of all
    buckets in bucket order (the piece table is in `flat_index`), and, with expert parallelism, `*.local`
    of shape [world * local_numel]. Every rank writes its own chunk files; nothing crosses the ranks."""
    from ..ckpt.orbax_layout import ShardedArray
    out: Dict[Tuple, Any] = {("count", "value"): torch.as_tensor(state["count"])}
    for k in ("mu", "nu", "master"):
      out[(k, "flat", "value")] = ShardedArray(state[k]["flat"], (self.world * self.shard_numel,), (self.shard_numel,),
                                               (self.rank,))
      if "local" in state[k]:
        out[(k, "local", "value")] = ShardedArray(state[k]["local"], (self.world * self.local_numel,),
                                                  (self.local_numel,), (self.rank,))
    for n, v in (state.get("hyperparams") or {}).items():
      out[("hyperparams", n, "value")] = torch.as_tensor(v)
    return out

  def flat_index(self) -> Dict[str, Any]:
    """Where each parameter sits in the flat index space and which flat ranges each rank's chunk of the
    `state_shards` arrays holds (JSON-serialisable)."""
    per_rank = []
    for r in range(self.world):
      so, rows = 0, []
      for lo, n in self.buckets:
        per = n // self.world
        rows.append([lo + r * per, per, r * self.shard_numel + so])     # flat start, length, position in the array
        so += per
      per_rank.append(rows)
    return {"format": "tunix_b200.flat_state.v2", "numel": self.numel, "used": self.used, "world": self.world,
            "shard_numel": self.shard_numel, "pieces": per_rank, "names": list(self.names),
            "offsets": [self.offsets[n] for n in self.names], "shapes": [list(self.shapes[n]) for n in self.names],
            "local_numel": self.local_numel, "local_names": list(self.local_names),
            "local_offsets": [self.local_offsets[n] for n in self.local_names],
            "local_shapes": [list(self.local_shapes[n]) for n in self.local_names]}

  @torch.no_grad()
  def load_state_shards(self, state: Dict[str, Any], index: Mapping[str, Any], read_rows) -> None:
    """Restores this rank's shard from arrays written by `state_shards`, possibly by a job of another
    size: `read_rows(name, lo, hi)` returns elements [lo, hi) of the stored 1-D array `name`. Every piece
    this rank owns is assembled from the saved pieces that overlap it in the flat index space (parameter
    offsets do not depend on the number of ranks)."""
    if list(index["names"]) != list(self.names) or list(index["offsets"]) != [self.offsets[n] for n in self.names]:
      raise ValueError("checkpointed optimizer state was written for a different parameter layout")
    saved = [tuple(p) for rows in index["pieces"] for p in rows]       # (flat start, length, array position)
    for k in ("mu", "nu", "master"):
      dst = state[k]["flat"]
      for lo, n, so in self.pieces:
        for flo, fn, pos in saved:
          a, b = max(lo, flo), min(lo + n, flo + fn)
          if a < b:
            part = read_rows(f"{k}.flat", pos + (a - flo), pos + (b - flo))
            dst[so + (a - lo): so + (b - lo)].copy_(part.to(self.device, torch.float32))
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
    parts = torch.empty(self.world * self.shard_numel, dtype=shard_tensor.dtype, device=shard_tensor.device)
    dist.all_gather_into_tensor(parts, shard_tensor.contiguous(), group=self.group)
    full = torch.zeros(self.numel, dtype=shard_tensor.dtype, device=shard_tensor.device)
    for r in range(self.world):                    # rank-major pieces back into flat order
      so = 0
      for lo, n in self.buckets:
        per = n // self.world
        full[lo + r * per: lo + (r + 1) * per].copy_(parts[r * self.shard_numel + so: r * self.shard_numel + so + per])
        so += per
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
      state[k]["flat"].copy_(self._my_part(full))
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
    state["master"]["flat"].copy_(self._my_part(self.flat_param).float())
    if "local" in state["master"]:
      state["master"]["local"].copy_(self.local_param.float())


def shard_model(model: torch.nn.Module, mesh: Optional[mesh_lib.Mesh] = None, axis: str = "fsdp",
                transport: Optional[str] = None, mode: Optional[str] = None) -> torch.nn.Module:
  """Moves the trainable parameters of `model` into a `FlatParamStore` (attached as
  `model.flat_store`). With `mesh=None` the store is single-rank: same flat layout, fused
  one-kernel optimizer step, no communication. All ranks must start from identical weights
  (same seed) or call `broadcast_params` afterwards. `mode="sharded"` (or `TUNIX_FSDP_MODE=sharded`) shards the
  decoder layers' parameters and gradients too (`fsdp_sharded.ShardedParamStore`)."""
  mode = mode or os.environ.get("TUNIX_FSDP_MODE", "resident")
  if mode == "sharded":
    from . import fsdp_sharded
    return fsdp_sharded.shard_model(model, mesh, axis)
  if mode != "resident":
    raise ValueError(f"unknown FSDP mode {mode!r}: 'resident' or 'sharded'")
  store = FlatParamStore(model, mesh, axis, transport)
  model.flat_store = store
  return model


def broadcast_params(model: torch.nn.Module, src: int = 0) -> None:
  store: FlatParamStore = model.flat_store
  if store.world == 1:
    return
  ranks = store.mesh.ranks()
  if store.resident:
    dist.broadcast(store.flat_param, src=ranks[src], group=store.mesh.all_group())
    return
  with store.summon_full_params(writeback=True):
    for p in store.params.values():
      dist.broadcast(p.data, src=ranks[src], group=store.mesh.all_group())


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
