"""Transport-neutral weight-sync protocol (tunix/experimental/orchestrator/weight_sync.py:34-373).

The coordinator moves no bytes. Sources and destinations describe what they hold as
`WorkUnitMetadata` (plain Python data: identity, data-plane addresses, per-tensor shape /
sharding), a `WeightSyncHandler` registers those units and executes `transfer(src, dst)`.
On this platform the default handler copies through NVLink peer memory
(`peer_memory_handler.PeerMemoryHandler`); an in-process handler serves tests.

Source side of a round: `prepare_weight_sync` (stage this version, return its metadata) and
`release_weight_sync`. Destination side: `bind_weight_sync` (transport resources, while still
serving), `get_weight_sync_metadata`, `pre_weight_sync` (stop admitting, drain, free KV
cache), `weight_sync` (materialise into STAGING only), `post_weight_sync` (atomic publish,
rebuild cache, resume), `abort_weight_sync` (drop staging, resume on the old weights) and
`get_weight_sync_status`. Rollback is possible only because `weight_sync` never touches the
serving copy.
"""
from __future__ import annotations

import abc
import dataclasses
from typing import Any, Optional, Protocol, Sequence, Tuple, runtime_checkable


@dataclasses.dataclass(frozen=True)
class WorkUnitId:
  job_name: str
  job_replica_id: str = ""
  data_name: str = ""
  data_replica_idx: int = 0

  def __post_init__(self):
    if not self.job_name:
      raise ValueError("work-unit job_name must not be empty")
    if self.data_replica_idx < 0:
      raise ValueError("work-unit data_replica_idx must be non-negative")


@dataclasses.dataclass(frozen=True)
class TensorMetadata:
  """One tensor of a work unit. `sharding_spec` names one mesh axis per tensor dimension
  ("" = replicated along it); `mesh_shape` is the logical per-dimension split; `layout` is
  minor-to-major order; `layer_idx` is a batching ordinal transports may use."""
  name: str
  shape: Tuple[int, ...]
  mesh_shape: Tuple[int, ...]
  layout: Tuple[int, ...]
  item_size: int
  layer_idx: int = 0
  sharding_spec: Tuple[str, ...] = ()

  def __post_init__(self):
    rank = len(self.shape)
    if not self.name:
      raise ValueError("variable name must not be empty")
    if not self.shape or any(d <= 0 for d in self.shape):
      raise ValueError(f"variable {self.name!r} has invalid shape {self.shape}")
    if len(self.mesh_shape) != rank or any(d <= 0 for d in self.mesh_shape):
      raise ValueError(f"variable {self.name!r}: mesh_shape {self.mesh_shape} must have rank {rank} and positive "
                       "dimensions")
    if len(self.layout) != rank:
      raise ValueError(f"variable {self.name!r}: layout {self.layout} must have rank {rank}")
    if self.item_size <= 0:
      raise ValueError(f"variable {self.name!r}: item_size must be positive, got {self.item_size}")
    if self.layer_idx < 0:
      raise ValueError(f"variable {self.name!r}: layer_idx must be non-negative")
    if self.sharding_spec and len(self.sharding_spec) != rank:
      raise ValueError(f"variable {self.name!r}: sharding_spec {self.sharding_spec} must have rank {rank}")
    named = [a for a in self.sharding_spec if a]
    if len(named) != len(set(named)):
      raise ValueError(f"variable {self.name!r}: a mesh axis may not shard two tensor dimensions: {self.sharding_spec}")


@dataclasses.dataclass(frozen=True)
class WorkUnitMetadata:
  unit: WorkUnitId
  shards: Tuple[str, ...] = ()                 # data-plane addresses, one per shard
  control_plane_rpc_address: str = ""
  global_shape: Optional[Tuple[int, ...]] = None
  mesh_shape: Optional[Tuple[int, ...]] = None
  layout: Optional[Tuple[int, ...]] = None
  item_size: Optional[int] = None
  variables: Tuple[TensorMetadata, ...] = ()
  mesh_axes: Optional[Tuple[str, ...]] = None


@dataclasses.dataclass(frozen=True)
class TransferResult:
  req_id: str
  success: bool
  message: str = ""


class TransferOutcomeUnknownError(RuntimeError):
  """The transfer call's outcome is unknown (not known-failed): it may still be writing into
  destination staging. Treated like a transfer deadline: no rollback, no source release."""


class WeightSyncHandler(abc.ABC):
  @abc.abstractmethod
  def register_work_unit(self, metadata: WorkUnitMetadata) -> None:
    """Replace-by-id registration; both sides re-register every round."""

  @abc.abstractmethod
  def transfer(self, src_units: Sequence[WorkUnitId], dst_units: Sequence[WorkUnitId], req_id: Optional[str] = None,
               generation: Optional[int] = None) -> TransferResult: ...

  def close(self) -> None:
    return None


@runtime_checkable
class WeightSyncSource(Protocol):
  async def prepare_weight_sync(self, sync_request: Any = None, **kwargs: Any) -> Sequence[WorkUnitMetadata]: ...
  async def release_weight_sync(self, sync_request: Any = None, **kwargs: Any) -> Any: ...


@runtime_checkable
class WeightSyncDestination(Protocol):
  async def bind_weight_sync(self) -> None: ...
  async def get_weight_sync_metadata(self) -> Sequence[WorkUnitMetadata]: ...
  async def pre_weight_sync(self, sync_request: Any = None) -> Any: ...
  async def weight_sync(self, sync_request: Any = None) -> Any: ...
  async def post_weight_sync(self, sync_request: Any = None) -> Any: ...
  async def abort_weight_sync(self, sync_request: Any = None) -> Any: ...
  async def get_weight_sync_status(self) -> Any: ...
