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


def _fail_unless(ok: bool, what: str) -> None:
  if not ok:
    raise ValueError(what)


@dataclasses.dataclass(frozen=True)
class WorkUnitId:
  """Names one transferable unit: the job that owns it (trainer, a rollout replica), which replica of
  that job, which named piece of data, and which data-parallel copy of that piece."""
  job_name: str
  job_replica_id: str = ""
  data_name: str = ""
  data_replica_idx: int = 0

  def __post_init__(self):
    _fail_unless(bool(self.job_name), "a work unit needs the name of the job that owns it")
    _fail_unless(self.data_replica_idx >= 0, f"data_replica_idx is an index, got {self.data_replica_idx}")


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
    _fail_unless(bool(self.name), "a tensor record needs a name")
    nd, who = len(self.shape), f"tensor {self.name!r}"
    axes = [a for a in self.sharding_spec if a]
    # (condition that must hold, complaint) - evaluated in order, the first broken one is reported
    rules = (
        (nd > 0 and min(self.shape) > 0, f"{who}: every extent of shape {self.shape} must be at least 1"),
        (len(self.mesh_shape) == nd, f"{who}: mesh_shape {self.mesh_shape} does not have the tensor's rank {nd}"),
        (all(m > 0 for m in self.mesh_shape), f"{who}: mesh_shape {self.mesh_shape} has a non-positive split"),
        (len(self.layout) == nd, f"{who}: layout {self.layout} does not have the tensor's rank {nd}"),
        (self.item_size > 0, f"{who}: item_size {self.item_size} is not a byte count"),
        (self.layer_idx >= 0, f"{who}: layer_idx {self.layer_idx} is not an ordinal"),
        (not self.sharding_spec or len(self.sharding_spec) == nd,
         f"{who}: sharding_spec {self.sharding_spec} does not have the tensor's rank {nd}"),
        (len(axes) == len(set(axes)), f"{who}: sharding_spec {self.sharding_spec} uses one mesh axis for two tensor "
                                      "dimensions"),
    )
    for holds, complaint in rules:
      _fail_unless(holds, complaint)


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
  """The data plane. Implementations move bytes; the coordinator only tells them which units."""

  @abc.abstractmethod
  def register_work_unit(self, metadata: WorkUnitMetadata) -> None:
    """Records (or replaces, by id) what a unit looks like; both sides re-register every round."""

  @abc.abstractmethod
  def transfer(self, src_units: Sequence[WorkUnitId], dst_units: Sequence[WorkUnitId], req_id: Optional[str] = None,
               generation: Optional[int] = None) -> TransferResult:
    """Copies the source units into the destinations' STAGING storage and reports the outcome."""

  def close(self) -> None:
    return None


# The calls of one round, in the order the coordinator issues them. A participant implements the
# side(s) it plays; the coordinator checks by duck typing (`runtime_checkable`), so a remote handle
# that forwards these names over RPC qualifies as well as a local object.
SOURCE_PHASES = ("prepare_weight_sync", "release_weight_sync")
DESTINATION_PHASES = ("bind_weight_sync", "get_weight_sync_metadata", "pre_weight_sync", "weight_sync",
                      "post_weight_sync", "abort_weight_sync", "get_weight_sync_status")


@runtime_checkable
class WeightSyncSource(Protocol):
  """Holder of the new weights."""

  async def prepare_weight_sync(self, sync_request: Any = None, **kwargs: Any) -> Sequence[WorkUnitMetadata]:
    """Pins the version named by the request and describes it; nothing may overwrite it until release."""

  async def release_weight_sync(self, sync_request: Any = None, **kwargs: Any) -> Any:
    """The round is over (either way): the pinned version may be dropped."""


@runtime_checkable
class WeightSyncDestination(Protocol):
  """Receiver of the new weights; keeps serving the old ones until `post_weight_sync`."""

  async def bind_weight_sync(self) -> None:
    """Sets up transport resources (staging buffers, peer mappings) while still serving."""

  async def get_weight_sync_metadata(self) -> Sequence[WorkUnitMetadata]:
    """Describes the staging units the transport should fill."""

  async def pre_weight_sync(self, sync_request: Any = None) -> Any:
    """Stops admitting requests, drains those in flight, frees what the new weights invalidate."""

  async def weight_sync(self, sync_request: Any = None) -> Any:
    """Materialises the transferred bytes - into staging only, never into the serving copy."""

  async def post_weight_sync(self, sync_request: Any = None) -> Any:
    """Publishes staging as the serving copy in one step, rebuilds caches, resumes admission."""

  async def abort_weight_sync(self, sync_request: Any = None) -> Any:
    """Drops staging and resumes on the old weights."""

  async def get_weight_sync_status(self) -> Any:
    """Which version is served and whether a round is in progress."""
