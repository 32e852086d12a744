"""Fully sharded data parallel training with sharded PARAMETERS: the mode for models whose bf16 replica plus fp32
gradient buffer do not fit beside the activations (Llama-70B class on 180 GB GPUs).

The resident store (`fsdp.FlatParamStore`) keeps the whole bf16 model and a whole fp32 gradient buffer on every rank
and shards only what the optimizer touches. Here the decoder layers - nearly all of a model - exist on a rank only
as its 1/world slice (bf16 compute copy, fp32 gradient accumulator, fp32 master and both Adam moments); a layer is
whole on a GPU only while it computes. (The reference shards parameters on the 'fsdp' mesh axis and lets the compiler
place the gathers, tunix/models/llama3/model.py:65-82, tunix/sft/peft_trainer.py:636-677.)

Units. The flat index space and its buckets are the resident store's (so checkpoints, `state_shards` and
`flat_index` are interchangeable between the two modes); a *unit* is a bucket made of decoder layers, by default one
layer (`TUNIX_FSDP_SHARDED_UNIT_LAYERS`). What precedes and follows the layers (embedding, final norm, head: 2 of
8 B parameters for Llama-3.1-8B) stays resident as in the other store, because the loss reads the head outside any
layer call.

Life of a unit during one micro-batch:

  forward   a pre-forward hook on the unit's first layer makes the unit whole: all-gather of the ranks' bf16 slices
            into one of two rotating slots (slot = unit index mod 2, so a unit always lands on the same addresses),
            parameters re-pointed at views of the slot; the NEXT unit's gather is issued right away on a side stream
            into the other slot and overlaps this unit's compute;
  backward  a hook on the unit's output gradient makes it whole again (the previous unit in backward order is
            prefetched), points every parameter's `main_grad` at a zeroed fp32 gradient slot, and, when the backward
            pass has moved on to the next unit, the slot is reduce-scattered on the side stream and ADDED into this
            rank's persistent fp32 gradient slice. No full gradient buffer ever exists.

The optimizer step then has nothing left to reduce but the resident buckets: global norm over the slices, fused AdamW
on the slice (bf16 slice refreshed in place), all-gather of the resident buckets only.

Stream discipline (CUDA): a slot is written by the side stream only after an event recorded on the compute stream
when the slot's previous user had been enqueued; the compute stream waits for the gather's event before the unit's
first kernel. On CPU (gloo ranks in tests) everything is synchronous.

Limits, stated rather than hidden: per-block activation recomputation is supported (the recomputation runs inside
the unit's backward window), whole-decoder recomputation is not; expert-parallel parameters are not; code that reads
layer weights outside a layer's `forward` (the paged rollout engine, exporters) must do so inside
`summon_full_params()`; the model is built whole on the device before it is sharded.
"""
from __future__ import annotations

import contextlib
import functools
import os
from typing import Any, Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

from . import fsdp


def _in_backward() -> bool:
  probe = getattr(torch._C, "_current_graph_task_id", None)
  return probe is not None and probe() != -1


class _Unit:
  """One on-demand bucket: where it sits in the flat space and in the shard, and its parameters."""

  def __init__(self, bucket: int, index: int, lo: int, numel: int, shard_off: int, per: int):
    self.bucket, self.index, self.lo, self.numel, self.shard_off, self.per = bucket, index, lo, numel, shard_off, per
    self.params: List[Tuple[torch.nn.Parameter, int, Tuple[int, ...]]] = []    # (parameter, offset in unit, shape)
    self.ready: Optional[torch.cuda.Event] = None      # the gather that filled this unit's slot


class ShardedParamStore(fsdp.FlatParamStore):
  resident = False

  def _layers_per_bucket(self) -> int:
    return int(os.environ.get("TUNIX_FSDP_SHARDED_UNIT_LAYERS", "1"))

  # ---- construction ----------------------------------------------------------------------------
  def _allocate(self, model: torch.nn.Module, params, local, transport: Optional[str]) -> None:
    if local:
      raise NotImplementedError("sharded-parameter mode does not take expert-parallel parameters")
    ids = self._bucket_ids
    if ids is None:
      raise ValueError("sharded-parameter mode needs per-layer buckets: a power-of-two number of ranks (<= 16) and "
                       "parameters in layer order")
    dev, dtype = self.device, self.dtype
    self.transport = "nccl" if dev.type == "cuda" else "gloo"
    self.symm = None
    self.local_param = self.local_grad = None
    self.local_names, self.local_shapes, self.local_offsets, self.local_numel = [], {}, {}, 0
    self.params = dict(params)
    # bucket number of every parameter, in flat order
    bucket_of: Dict[str, int] = {}
    b, last = -1, None
    for i, (n, _) in enumerate(params):
      if ids[i] != last:
        b, last = b + 1, ids[i]
      bucket_of[n] = b
    layer_buckets = {bucket_of[n] for n, _ in params if fsdp._layer_index(n) is not None}
    self.units: List[_Unit] = []
    self._unit_of_bucket: Dict[int, _Unit] = {}
    for bi, ((lo, bn), (_, per, so)) in enumerate(zip(self.buckets, self.pieces)):
      if bi in layer_buckets:
        u = _Unit(bi, len(self.units), lo, bn, so, per)
        self.units.append(u)
        self._unit_of_bucket[bi] = u
    if not self.units:
      raise ValueError("model has no decoder layers to shard")
    self.param_shard = torch.zeros(self.shard_numel, dtype=dtype, device=dev)
    self.grad_shard = torch.zeros(self.shard_numel, dtype=torch.float32, device=dev)
    widest = max(u.numel for u in self.units)
    self._slots = [torch.zeros(widest, dtype=dtype, device=dev) for _ in range(2)]
    self._grad_slots = [torch.zeros(widest, dtype=torch.float32, device=dev) for _ in range(2)]
    self._held: List[Optional[int]] = [None, None]          # unit index whose gathered values a slot holds
    self._grad_free: List[Optional[Any]] = [None, None]     # event: the slot's last reduce-scatter has read it
    self._open: Optional[_Unit] = None                      # unit whose gradient slot is collecting
    self._comm = torch.cuda.Stream(device=dev) if dev.type == "cuda" else None
    self._piece_tmp = torch.zeros(max(u.per for u in self.units), dtype=torch.float32, device=dev)
    self._tmp_free = None
    # resident buckets: whole bf16 values and whole fp32 gradients, as in the resident store
    self._resident: Dict[int, Tuple[torch.Tensor, torch.Tensor]] = {}
    for bi, (lo, bn) in enumerate(self.buckets):
      if bi not in layer_buckets:
        self._resident[bi] = (torch.zeros(bn, dtype=dtype, device=dev), torch.zeros(bn, dtype=torch.float32, device=dev))
    with torch.no_grad():
      for n, p in params:
        bi, o, numel = bucket_of[n], self.offsets[n], p.numel()
        lo, bn = self.buckets[bi]
        per = bn // self.world
        if bi in self._resident:
          values, grads = self._resident[bi]
          view = values[o - lo:o - lo + numel].view(p.shape)
          view.copy_(p.data)
          p.data = view
          p.main_grad = grads[o - lo:o - lo + numel].view(p.shape)
        else:
          u = self._unit_of_bucket[bi]
          u.params.append((p, o - lo, tuple(p.shape)))
          # this rank's slice of the parameter's values goes into the persistent shard
          mine_lo, mine_hi = lo + self.rank * per, lo + (self.rank + 1) * per
          a, z = max(o, mine_lo), min(o + numel, mine_hi)
          if a < z:
            self.param_shard[u.shard_off + (a - mine_lo): u.shard_off + (z - mine_lo)].copy_(
                p.data.reshape(-1)[a - o: z - o])
          p.main_grad = None
          p.grad_managed = True         # the trainer's accumulator leaves this parameter's gradients to the store
      for bi, (values, _) in self._resident.items():
        lo, n, so = self.pieces[bi]
        blo = self.buckets[bi][0]
        self.param_shard[so:so + n].copy_(values[lo - blo: lo - blo + n])
      for u in self.units:              # original storage is released; values come back with the first gather
        self._bind(u, self._slots[u.index % 2])
    self._install_unit_hooks(model)
    # attributes of the resident store's overlap machinery that shared code looks at
    self._reduced, self._armed, self._side = set(), False, None
    self._scratch: Dict[str, torch.Tensor] = {}
    self._bucket_of_layer, self._layers_in_bucket = {}, {}
    model.gather_for_checkpoint = functools.partial(self._checkpoint_tree, model)
    model.scatter_from_checkpoint = functools.partial(self._load_checkpoint_tree, model)

  @property
  def flat_param(self):
    raise AttributeError("a sharded-parameter store has no whole parameter buffer; use summon_full_params()")

  @property
  def flat_grad(self):
    raise AttributeError("a sharded-parameter store has no whole gradient buffer")

  def _bind(self, unit: _Unit, slot: torch.Tensor) -> None:
    for p, o, shape in unit.params:
      p.data = slot[o:o + p.numel()].view(shape)

  def _install_unit_hooks(self, model: torch.nn.Module) -> None:
    layers = getattr(model, "layers", None)
    if layers is None:
      raise ValueError("sharded-parameter mode needs a model with a `layers` list")
    by_unit: Dict[int, List[torch.nn.Module]] = {}
    for i, layer in enumerate(layers):
      own = {id(p) for p in layer.parameters()}
      for u in self.units:
        if any(id(p) in own for p, _, _ in u.params):
          by_unit.setdefault(u.index, []).append(layer)
          break
    for ui, members in by_unit.items():
      u = self.units[ui]
      members[0].register_forward_pre_hook(functools.partial(self._before_forward, u))
      members[-1].register_forward_hook(functools.partial(self._after_forward, u))

  # ---- collectives -----------------------------------------------------------------------------
  def _all_gather(self, dst: torch.Tensor, src: torch.Tensor) -> None:
    if self.world == 1:
      dst.copy_(src)
    else:
      dist.all_gather_into_tensor(dst, src, group=self.group)

  def _reduce_scatter(self, dst: torch.Tensor, src: torch.Tensor) -> None:
    """dst[per] = sum over ranks of src[rank * per: (rank + 1) * per]."""
    per = dst.numel()
    if self.world == 1:
      dst.copy_(src[:per])
    elif self.device.type == "cuda":
      dist.reduce_scatter_tensor(dst, src, op=dist.ReduceOp.SUM, group=self.group)
    else:
      dist.all_reduce(src, op=dist.ReduceOp.SUM, group=self.group)      # gloo has no reduce-scatter
      dst.copy_(src[self.rank * per:(self.rank + 1) * per])

  # ---- making a unit whole ---------------------------------------------------------------------
  def _issue_gather(self, unit: _Unit) -> None:
    """All-gather of the unit's slices into its slot, on the side stream, after everything enqueued so far on the
    compute stream (which includes the slot's previous user)."""
    slot = self._slots[unit.index % 2]
    src = self.param_shard[unit.shard_off:unit.shard_off + unit.per]
    if self._comm is None:
      self._all_gather(slot[:unit.numel], src)
    else:
      here = torch.cuda.current_stream(self.device)
      enqueued = torch.cuda.Event()
      enqueued.record(here)
      with torch.cuda.stream(self._comm):
        self._comm.wait_event(enqueued)
        self._all_gather(slot[:unit.numel], src)
        unit.ready = torch.cuda.Event()
        unit.ready.record(self._comm)
    self._held[unit.index % 2] = unit.index

  def _ensure(self, unit: _Unit, direction: int) -> None:
    """The unit is whole and bound when this returns (on the compute stream's timeline); its neighbour in
    `direction` is on its way into the other slot."""
    if self._held[unit.index % 2] != unit.index:
      self._issue_gather(unit)
    if unit.ready is not None:
      torch.cuda.current_stream(self.device).wait_event(unit.ready)
      unit.ready = None
    self._bind(unit, self._slots[unit.index % 2])
    nxt = unit.index + direction
    if self._comm is not None and 0 <= nxt < len(self.units) and self._held[nxt % 2] != nxt:
      self._issue_gather(self.units[nxt])

  # ---- hooks -----------------------------------------------------------------------------------
  def _before_forward(self, unit: _Unit, module, args) -> None:
    if _in_backward():
      if self._open is not unit:
        raise RuntimeError("sharded-parameter mode supports per-block recomputation only: a layer outside the "
                           "unit in backward was asked to recompute")
      return                      # recomputation of the unit in backward: already whole
    self._finish_backward()       # a new forward pass: the previous backward pass is over
    self._ensure(unit, +1)

  def _after_forward(self, unit: _Unit, module, args, output) -> None:
    if _in_backward() or not torch.is_grad_enabled():
      return
    h = output[0] if isinstance(output, (tuple, list)) else output
    if isinstance(h, torch.Tensor) and h.requires_grad:
      h.register_hook(functools.partial(self._enter_backward, unit))

  def _enter_backward(self, unit: _Unit, grad: torch.Tensor) -> None:
    """The gradient of the unit's output exists: its backward (and recomputation) runs next."""
    if self._open is unit:
      return
    self._finish_backward()
    self._ensure(unit, -1)
    gslot = self._grad_slots[unit.index % 2]
    free = self._grad_free[unit.index % 2]
    if free is not None:
      torch.cuda.current_stream(self.device).wait_event(free)
      self._grad_free[unit.index % 2] = None
    gslot[:unit.numel].zero_()
    for p, o, shape in unit.params:
      p.main_grad = gslot[o:o + p.numel()].view(shape)
    self._open = unit

  @torch.no_grad()
  def _finish_backward(self) -> None:
    """Closes the unit whose gradients were collecting: folds gradients that arrived through `.grad`, then
    reduce-scatters the slot and adds this rank's part into the persistent gradient slice."""
    unit = self._open
    if unit is None:
      return
    self._open = None
    gslot = self._grad_slots[unit.index % 2]
    for p, o, shape in unit.params:
      if p.grad is not None:
        p.main_grad.add_(p.grad.to(torch.float32))
        p.grad = None
      p.main_grad = None
    mine = self.grad_shard[unit.shard_off:unit.shard_off + unit.per]
    if self._comm is None:
      tmp = self._piece_tmp[:unit.per]
      self._reduce_scatter(tmp, gslot[:unit.numel])
      mine.add_(tmp)
      return
    here = torch.cuda.current_stream(self.device)
    written = torch.cuda.Event()
    written.record(here)
    with torch.cuda.stream(self._comm):
      self._comm.wait_event(written)
      tmp = self._piece_tmp[:unit.per]
      self._reduce_scatter(tmp, gslot[:unit.numel])
      mine.add_(tmp)                    # side stream only ever touches grad_shard between optimizer steps
      done = torch.cuda.Event()
      done.record(self._comm)
    self._grad_free[unit.index % 2] = done

  def after_backward(self) -> None:
    """Called by the trainer when a backward pass has returned: the last unit's reduction can start now instead
    of at the next forward pass."""
    self._finish_backward()

  def arm_overlap(self) -> None:      # reductions of this mode always overlap; nothing to arm
    return

  # ---- optimizer step --------------------------------------------------------------------------
  def init_state(self, tx) -> Dict[str, Any]:
    master = self.param_shard.float()
    st: Dict[str, Any] = {"count": torch.zeros((), dtype=torch.int32), "master": {"flat": master},
                          "mu": {"flat": torch.zeros_like(master)}, "nu": {"flat": torch.zeros_like(master)}}
    if getattr(tx, "exposes_hyperparams", False):
      from .. import optim
      st["hyperparams"] = {"learning_rate": torch.tensor(optim._lr_at(tx._lr, 0), dtype=torch.float32)}
    return st

  @torch.no_grad()
  def step(self, tx, state: Dict[str, Any], denom: torch.Tensor, max_grad_norm: Optional[float]) -> torch.Tensor:
    self._finish_backward()
    if self._comm is not None:
      torch.cuda.current_stream(self.device).wait_stream(self._comm)
    d = self._buf("denom")
    d.copy_(denom.reshape(1))
    ss = self._buf("sumsq")
    for bi, (_, grads) in self._resident.items():
      _, n, so = self.pieces[bi]
      self._reduce_scatter(self.grad_shard[so:so + n], grads)
    norm, scale = self._norm_and_scale(self.grad_shard, ss, d, max_grad_norm)
    inner = getattr(tx, "inner", tx)
    inner.fused_flat_step(state["master"]["flat"], state["mu"]["flat"], state["nu"]["flat"], self.grad_shard,
                          self.param_shard, state, scale, zero_grad=False)
    for bi, (values, grads) in self._resident.items():
      _, n, so = self.pieces[bi]
      self._all_gather(values, self.param_shard[so:so + n])
      grads.zero_()
    self.grad_shard.zero_()
    self._held = [None, None]           # gathered copies are of the old values
    return norm[0].clone()

  @torch.no_grad()
  def refresh_master_from_params(self, state: Dict[str, Any]) -> None:
    state["master"]["flat"].copy_(self.param_shard.float())

  # ---- whole-model access ----------------------------------------------------------------------
  @contextlib.contextmanager
  def summon_full_params(self, writeback: bool = False):
    """Inside the block every parameter is whole on every rank (temporary buffers: the memory of a bf16
    replica). With `writeback` the values found at exit become the model: every rank keeps its slice of them
    (the ranks must have written the same values)."""
    self._finish_backward()
    whole = []
    with torch.no_grad():
      for u in self.units:
        buf = torch.empty(u.numel, dtype=self.dtype, device=self.device)
        self._all_gather(buf, self.param_shard[u.shard_off:u.shard_off + u.per])
        self._bind(u, buf)
        whole.append(buf)
    try:
      yield self
    finally:
      with torch.no_grad():
        for u, buf in zip(self.units, whole):
          if writeback:
            self.param_shard[u.shard_off:u.shard_off + u.per].copy_(buf[self.rank * u.per:(self.rank + 1) * u.per])
          self._bind(u, self._slots[u.index % 2])
        if writeback:
          for bi, (values, _) in self._resident.items():
            lo, n, so = self.pieces[bi]
            blo = self.buckets[bi][0]
            self.param_shard[so:so + n].copy_(values[lo - blo: lo - blo + n])
        self._held = [None, None]

  def _checkpoint_tree(self, model: torch.nn.Module, lora_only: bool = False):
    """Checkpoint tree of the whole model, on the host (the checkpoint writer's `gather_for_checkpoint` hook)."""
    from ..ckpt import layout
    with self.summon_full_params():
      tree = layout.model_to_tree(model, lora_only)
      keep = self.rank == 0
      return {k: (v.detach().to("cpu", copy=True) if keep else v.detach().new_empty(0)) for k, v in tree.items()}

  def _load_checkpoint_tree(self, model: torch.nn.Module, tree, lora_only: bool = False, **kwargs) -> None:
    from ..ckpt import layout
    with self.summon_full_params(writeback=True):
      layout.tree_to_model(model, tree, lora_only, **kwargs)

  def memory_report(self) -> Dict[str, float]:
    """GB held by the store on this rank, by kind."""
    gb = lambda t: t.numel() * t.element_size() / 1e9   # noqa: E731
    res = sum(gb(v) + gb(g) for v, g in self._resident.values())
    return {"param_shard": gb(self.param_shard), "grad_shard": gb(self.grad_shard),
            "slots": sum(gb(s) for s in self._slots) + sum(gb(s) for s in self._grad_slots), "resident": res}


def shard_model(model: torch.nn.Module, mesh=None, axis: str = "fsdp") -> torch.nn.Module:
  """`fsdp.shard_model` with sharded parameters (attached as `model.flat_store` as well)."""
  model.flat_store = ShardedParamStore(model, mesh, axis)
  return model
