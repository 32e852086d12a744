"""Weight-sync transports for this platform (the role `RaidenHandler` has in the reference,
tunix/experimental/orchestrator/raiden_handler.py:49-550).

`InProcessHandler`: source and destination units live in one process; `transfer` copies the
registered source tensors into the registered destination staging tensors (device-to-device
`copy_`, which on one node is an NVLink peer copy when the tensors sit on different GPUs).
`PeerMemoryHandler`: the same contract across processes of one node; each work unit names a
rank, transfers run as `torch.distributed` broadcasts from the owning rank inside the job's
process group (NCCL over NVLink), one call per tensor in manifest order, so that every rank
executes the same sequence of collectives.
"""
from __future__ import annotations

import threading
from typing import Any, Dict, Mapping, Optional, Sequence

import torch

from . import weight_sync


def manifest_of(unit: weight_sync.WorkUnitId, tensors: Mapping[str, torch.Tensor], shards: Sequence[str] = ()
                ) -> weight_sync.WorkUnitMetadata:
  """Metadata of a set of (unsharded) tensors held by one process."""
  vars_ = tuple(weight_sync.TensorMetadata(name=n, shape=tuple(t.shape) or (1,), mesh_shape=(1,) * max(t.dim(), 1),
                                           layout=tuple(range(max(t.dim(), 1) - 1, -1, -1)), item_size=t.element_size(),
                                           layer_idx=i) for i, (n, t) in enumerate(tensors.items()))
  return weight_sync.WorkUnitMetadata(unit=unit, shards=tuple(shards), variables=vars_)


class InProcessHandler(weight_sync.WeightSyncHandler):
  def __init__(self):
    self._lock = threading.Lock()
    self._meta: Dict[weight_sync.WorkUnitId, weight_sync.WorkUnitMetadata] = {}
    self._tensors: Dict[weight_sync.WorkUnitId, Mapping[str, torch.Tensor]] = {}

  def attach(self, unit: weight_sync.WorkUnitId, tensors: Mapping[str, torch.Tensor]) -> None:
    """Gives the transport access to a unit's tensors (sources: the prepared weights;
    destinations: the staging copy)."""
    with self._lock:
      self._tensors[unit] = tensors

  def register_work_unit(self, metadata: weight_sync.WorkUnitMetadata) -> None:
    with self._lock:
      self._meta[metadata.unit] = metadata

  def _check(self, src: weight_sync.WorkUnitMetadata, dst: weight_sync.WorkUnitMetadata) -> Optional[str]:
    s = {v.name: v for v in src.variables}
    for v in dst.variables:
      if v.name not in s:
        return f"destination {dst.unit.job_name} expects {v.name!r}, which the source does not provide"
      if s[v.name].shape != v.shape:
        return f"shape mismatch for {v.name!r}: source {s[v.name].shape} vs destination {v.shape}"
    return None

  @torch.no_grad()
  def transfer(self, src_units, dst_units, req_id=None, generation=None) -> weight_sync.TransferResult:
    rid = req_id or ""
    with self._lock:
      if not src_units or not dst_units:
        return weight_sync.TransferResult(rid, False, "transfer needs at least one source and one destination unit")
      for u in list(src_units) + list(dst_units):
        if u not in self._meta:
          return weight_sync.TransferResult(rid, False, f"work unit {u} was never registered")
        if u not in self._tensors:
          return weight_sync.TransferResult(rid, False, f"work unit {u} has no tensors attached")
      src_u = src_units[0]
      for d in dst_units:
        err = self._check(self._meta[src_u], self._meta[d])
        if err:
          return weight_sync.TransferResult(rid, False, err)
      moved = 0
      for d in dst_units:
        dst_t = self._tensors[d]
        for name, t in dst_t.items():
          t.copy_(self._tensors[src_u][name].to(t.dtype), non_blocking=True)
          moved += t.numel() * t.element_size()
      if torch.cuda.is_available():
        torch.cuda.synchronize()
    return weight_sync.TransferResult(rid, True, f"{moved} bytes to {len(dst_units)} destination unit(s)")


class PeerMemoryHandler(InProcessHandler):
  """Multi-process variant: `data_replica_idx` of a unit is the global rank that owns it."""

  def __init__(self, group=None):
    super().__init__()
    self._group = group

  @torch.no_grad()
  def transfer(self, src_units, dst_units, req_id=None, generation=None) -> weight_sync.TransferResult:
    import torch.distributed as dist
    if not dist.is_initialized() or dist.get_world_size(self._group) == 1:
      return super().transfer(src_units, dst_units, req_id, generation)
    rid = req_id or ""
    me = dist.get_rank()
    src = src_units[0]
    names = [v.name for v in self._meta[src].variables]
    mine = [u for u in dst_units if u.data_replica_idx == me]
    moved = 0
    for name in names:                       # same order of collectives on every rank
      if me == src.data_replica_idx:
        buf = self._tensors[src][name]
      elif mine:
        buf = self._tensors[mine[0]][name]
      else:
        v = next(v for v in self._meta[src].variables if v.name == name)
        buf = torch.empty(v.shape, dtype=torch.bfloat16, device="cuda" if torch.cuda.is_available() else "cpu")
      dist.broadcast(buf, src=src.data_replica_idx, group=self._group)
      for extra in mine[1:]:
        self._tensors[extra][name].copy_(buf)
      moved += buf.numel() * buf.element_size()
    return weight_sync.TransferResult(rid, True, f"{moved} bytes broadcast from rank {src.data_replica_idx}")
