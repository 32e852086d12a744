"""Trainer -> rollout weight transfer across layouts.

The trainer holds its parameters GEMM-ready in one flat bf16 buffer (`dist.fsdp.FlatParamStore`:
data-parallel ranks, sharded optimizer state). A rollout replica may use another layout: tensor
parallel over `tp` ranks (rows of the fused q|k|v and gate|up projections, columns of the output
and down projections, KV heads replicated when there are fewer of them than ranks), optionally a
vocabulary-sharded head. The reference expresses this as a cross-mesh re-shard with per-engine
key / transpose mappings (tunix/rl/reshard.py:171-261, tunix/generate/utils.py:825-964); here it is

  * a *plan*: for every rollout parameter the 2-D blocks of the trainer's flat buffer that make it
    up (`build_plan`), computed once and kept on the device as fixed-size records,
  * one kernel launch per sync (`tx_reshard_copy`, `csrc/peer_comm.cu`) that walks the whole plan with
    16-byte loads and stores. A source address may be the flat buffer of ANOTHER rank, reached
    through its peer mapping over NVLink (`source_rank`), so a rollout rank pulls exactly the bytes
    of its slice straight out of a trainer rank's memory - no gather of full tensors, no staging
    through the host or through a collective library,
  * a version word written by the same stream after the copy, and optional double buffering: the
    copy fills the inactive buffer while the engine still decodes from the active one, then
    `RolloutReplica.activate()` swaps the parameter pointers (under the caller's rollout lock).

On CPU (tests, gloo ranks) the same plan is executed with tensor slicing.
"""
from __future__ import annotations

import ctypes
import dataclasses
import time
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

# (source row, source col, rows, cols, destination row): one block of a source parameter viewed as a 2-D
# array [rows_total, cols_total]; destination parameters are contiguous [dst_rows, cols].
Block = Tuple[int, int, int, int, int]


def tp_blocks(name: str, shape: Sequence[int], cfg, tp: int, r: int, shard_vocab: bool = False
              ) -> Tuple[Tuple[int, ...], List[Block]]:
  """Shape of rank r's slice of parameter `name` (full shape `shape`) under tensor parallelism of
  degree `tp`, and the source blocks it is made of. `cfg` is the full model's config."""
  N, K, H, Fh = cfg.num_heads, cfg.num_kv_heads, cfg.head_dim, cfg.hidden_dim
  shape = tuple(int(s) for s in shape)
  rows, cols = (shape[0], int(np.prod(shape[1:]))) if len(shape) > 1 else (1, shape[0])

  def row_sections(sections) -> Tuple[Tuple[int, ...], List[Block]]:
    """sections: (first row, rows per rank, index of the rank's part) per section, stacked in order."""
    blocks, dst = [], 0
    for first, per, idx in sections:
      if len(shape) > 1:
        blocks.append((first + idx * per, 0, per, cols, dst))
      else:                     # a bias vector: one row, a column range
        blocks.append((0, first + idx * per, 1, per, 0))
      dst += per
    if len(shape) > 1:
      return (dst,) + shape[1:], blocks
    # re-base the column blocks of a vector onto its packed destination
    out, off = [], 0
    for (_, c0, _, n, _) in blocks:
      out.append((0, c0, 1, n, off))
      off += n
    return (dst,), out

  if tp == 1:
    return shape, [(0, 0, rows, cols, 0)]
  kv_local = max(1, K // tp)                 # fewer KV heads than ranks: neighbouring ranks share a head
  kv_idx = r * K // tp if K >= tp else r // (tp // K)
  if name.endswith("attn.qkv_proj.w") or name.endswith("attn.qkv_proj.b"):
    return row_sections([(0, N // tp * H, r), (N * H, kv_local * H, kv_idx if K < tp else r),
                         ((N + K) * H, kv_local * H, kv_idx if K < tp else r)])
  if name.endswith("attn.o_proj.w"):
    per = N * H // tp
    return (shape[0], per), [(0, r * per, rows, per, 0)]
  if name.endswith("mlp.gate_up_proj.w"):
    return row_sections([(0, Fh // tp, r), (Fh, Fh // tp, r)])
  if name.endswith("mlp.down_proj.w"):
    per = Fh // tp
    return (shape[0], per), [(0, r * per, rows, per, 0)]
  if shard_vocab and name == "lm_head.w" and shape[0] % tp == 0:
    per = shape[0] // tp
    return (per,) + shape[1:], [(r * per, 0, per, cols, 0)]
  return shape, [(0, 0, rows, cols, 0)]


@dataclasses.dataclass
class Plan:
  """Copy plan of one rollout replica: per destination parameter its shape, its offset in the replica's
  flat buffer, and the blocks of the trainer's flat buffer that fill it."""
  names: List[str]
  shapes: Dict[str, Tuple[int, ...]]
  dst_offsets: Dict[str, int]
  numel: int
  # (source flat offset, destination flat offset, rows, cols, source ld, destination ld), elements
  segments: List[Tuple[int, int, int, int, int, int]]

  @property
  def bytes(self) -> int:
    return sum(s[2] * s[3] for s in self.segments) * 2


def build_plan(names: Sequence[str], src_shapes: Dict[str, Sequence[int]], src_offsets: Dict[str, int], cfg, tp: int,
               r: int, shard_vocab: bool = False) -> Plan:
  shapes, offs, segs, off = {}, {}, [], 0
  for n in names:
    full = tuple(src_shapes[n])
    cols_full = int(np.prod(full[1:])) if len(full) > 1 else full[0]
    shp, blocks = tp_blocks(n, full, cfg, tp, r, shard_vocab)
    dst_cols = int(np.prod(shp[1:])) if len(shp) > 1 else shp[0]
    shapes[n], offs[n] = shp, off
    for (r0, c0, nr, nc, d0) in blocks:
      if len(full) > 1:
        segs.append((src_offsets[n] + r0 * cols_full + c0, off + d0 * dst_cols, nr, nc, cols_full, dst_cols))
      else:
        segs.append((src_offsets[n] + c0, off + d0, 1, nc, cols_full, dst_cols))
    off += (int(np.prod(shp)) + 7) // 8 * 8
  return Plan(list(names), shapes, offs, off, segs)


def _pack_segments(plan: Plan, src_base: int, dst_base: int, device) -> Tuple[torch.Tensor, int]:
  """Device records for `tx_reshard_copy` (64 bytes each) and the number of work units."""
  rec = np.zeros((len(plan.segments), 8), dtype=np.int64)
  units = 0
  for i, (so, do, rows, cols, sld, dld) in enumerate(plan.segments):
    src, dst = src_base + so * 2, dst_base + do * 2
    vec = int(cols % 8 == 0 and sld % 8 == 0 and dld % 8 == 0 and src % 16 == 0 and dst % 16 == 0)
    rec[i] = (src, dst, rows, cols, sld, dld, units, vec)     # last int64 = {vec (low 32 bits), pad}
    units += rows * (cols // 8 if vec else cols)
  return torch.from_numpy(rec).to(device), units


class RolloutReplica:
  """A rollout copy of a trainer's model in tensor-parallel layout, refreshed by `sync()`.

  trainer_model: a `Transformer` whose parameters live in a `FlatParamStore` (`dist.fsdp.shard_model`).
  mesh / axis: the rollout mesh and its tensor-parallel axis (size 1: plain copy of the replica).
  source_rank: index (in the store's group) of the rank whose flat buffer is read; default: this rank's own
    resident replica (a local re-layout). Any other rank is read through its peer mapping over NVLink.
  double_buffer: keep two destination buffers so a sync can run while the engine still reads the other.
  """

  def __init__(self, trainer_model: torch.nn.Module, mesh=None, axis: str = "tp", source_rank: Optional[int] = None,
               shard_vocab: bool = False, skinny_exit: bool = True, double_buffer: bool = False):
    from ..models.transformer import Transformer
    from . import tp as tp_lib
    store = getattr(trainer_model, "flat_store", None)
    if store is None:
      raise ValueError("RolloutReplica needs a trainer model in a flat parameter store (dist.fsdp.shard_model)")
    self.store = store
    cfg = trainer_model.config
    self.tp = mesh.axis_size(axis) if mesh is not None else 1
    self.rank = mesh.axis_index(axis) if mesh is not None else 0
    group = mesh.group(axis) if mesh is not None else None
    N, K, Fh = cfg.num_heads, cfg.num_kv_heads, cfg.hidden_dim
    if N % self.tp or Fh % self.tp or (K % self.tp and self.tp % K):
      raise ValueError(f"heads {N}/{K} and hidden {Fh} do not divide over tp={self.tp}")
    if cfg.is_moe and self.tp > 1:
      raise NotImplementedError("tensor-parallel rollout covers dense layers")
    names = list(store.names)
    self.plan = build_plan(names, store.shapes, store.offsets, cfg, self.tp, self.rank, shard_vocab)
    dev = store.device
    self.device = dev
    self.buffers = [torch.zeros(self.plan.numel, dtype=store.dtype, device=dev)
                    for _ in range(2 if double_buffer else 1)]
    self.active = 0
    self.version = torch.zeros(1, dtype=torch.int32, device=dev)   # number of completed syncs
    self.versions_issued = 0
    local = cfg.replace(num_heads=N // self.tp, num_kv_heads=max(1, K // self.tp), hidden_dim=Fh // self.tp,
                        query_pre_attn_scalar=cfg.query_pre_attn_scalar, fused_layers=False)
    model = Transformer(local, device="meta")       # structure only: parameters become views of the buffers
    missing = [n for n, _ in model.named_parameters() if n not in self.plan.shapes]
    if missing:
      raise ValueError(f"trainer store lacks rollout parameters {missing[:3]} (frozen parameters are not in the store)")
    self._params: Dict[str, torch.nn.Parameter] = {}
    for n, p in list(model.named_parameters()):
      if tuple(p.shape) != tuple(self.plan.shapes[n]):
        raise ValueError(f"{n}: rollout shape {tuple(p.shape)} differs from the planned slice {self.plan.shapes[n]}")
      holder, _, leaf = n.rpartition(".")
      mod = model.get_submodule(holder) if holder else model
      new = torch.nn.Parameter(self._view(n, 0), requires_grad=False)
      mod._parameters[leaf] = new
      self._params[n] = new
    if self.tp > 1:
      if skinny_exit and dev.type == "cuda":
        ctx = tp_lib.SkinnyExitContext(group, dev, 128, cfg.embed_dim)
        model.tp_exit = ctx
      for layer in model.layers:
        layer.attn.qkv_proj = tp_lib._ColumnEntry(layer.attn.qkv_proj, group)
        layer.mlp.gate_up_proj = tp_lib._ColumnEntry(layer.mlp.gate_up_proj, group)
        if skinny_exit and dev.type == "cuda":
          layer.attn.o_proj = tp_lib.SkinnyRowExit(layer.attn.o_proj, group, ctx)
          layer.mlp.down_proj = tp_lib.SkinnyRowExit(layer.mlp.down_proj, group, ctx)
        else:
          layer.attn.o_proj = tp_lib._RowExit(layer.attn.o_proj, group)
          layer.mlp.down_proj = tp_lib._RowExit(layer.mlp.down_proj, group)
      tp_lib._finish_tp(model, local, cfg, group, self.tp, self.rank, False)
      if shard_vocab and model.lm_head is not None and cfg.vocab_size % self.tp == 0:
        model.lm_head.w.vocab_parallel = (group, self.rank * (cfg.vocab_size // self.tp))
    self.model = model.eval()
    for p in self.model.parameters():
      p.requires_grad_(False)
    # where the bytes come from
    self.source_rank = store.rank if source_rank is None else int(source_rank)
    if self.source_rank != store.rank:
      if store.symm is None:
        raise ValueError("reading another rank's replica needs the peer-memory transport of the flat store")
      self._src_base = store.symm.ptrs_for(store.flat_param)[self.source_rank]
    else:
      self._src_base = store.flat_param.data_ptr()
    self._records = None
    self.last_sync_ms: Optional[float] = None
    self._events = None

  def _view(self, name: str, which: int) -> torch.Tensor:
    o, shp = self.plan.dst_offsets[name], self.plan.shapes[name]
    return self.buffers[which][o:o + int(np.prod(shp))].view(shp)

  def _bind(self, which: int) -> None:
    """Points every parameter of the replica at its place in buffer `which`."""
    for n, p in self._params.items():
      p.data = self._view(n, which)
    self.active = which

  # ---- the transfer -----------------------------------------------------------------------
  @torch.no_grad()
  def sync(self, activate: bool = True) -> int:
    """Copies the trainer's current weights into the inactive buffer (the only one without double
    buffering) on the current stream; returns the version this sync will publish. With `activate` the
    parameter pointers are swapped right away (the caller holds whatever lock keeps the engine idle)."""
    target = (self.active + 1) % len(self.buffers)
    buf = self.buffers[target]
    self.versions_issued += 1
    if self.device.type != "cuda":
      t0 = time.perf_counter()
      src = self.store.flat_param
      for (so, do, rows, cols, sld, dld) in self.plan.segments:
        s2 = torch.as_strided(src, (rows, cols), (sld, 1), so)
        torch.as_strided(buf, (rows, cols), (dld, 1), do).copy_(s2)
      self.version.fill_(self.versions_issued)
      self.last_sync_ms = (time.perf_counter() - t0) * 1e3
    else:
      from ..ops import _lib
      lib = _lib.require()
      if self._records is None:
        self._records = {}
      if target not in self._records:
        self._records[target] = _pack_segments(self.plan, self._src_base, buf.data_ptr(), self.device)
      rec, units = self._records[target]
      e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
      e0.record()
      fn = _lib.declare("tx_reshard_copy", [ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_void_p,
                                            ctypes.c_int, ctypes.c_void_p])
      rc = fn(rec.data_ptr(), rec.shape[0], units, self.version.data_ptr(), self.versions_issued, _lib.stream_ptr())
      _lib.check_rc(rc, "tx_reshard_copy")
      e1.record()
      self._events = (e0, e1)
    if activate and target != self.active:
      self._bind(target)
    return self.versions_issued

  def activate(self) -> None:
    """Swaps the engine onto the buffer filled by the last `sync(activate=False)`."""
    target = (self.active + 1) % len(self.buffers)
    if target != self.active:
      self._bind(target)

  def sync_ms(self) -> Optional[float]:
    """Device time of the last sync (waits for it)."""
    if self._events is not None:
      self._events[1].synchronize()
      self.last_sync_ms = self._events[0].elapsed_time(self._events[1])
      self._events = None
    return self.last_sync_ms

  def completed_version(self) -> int:
    return int(self.version.item())
