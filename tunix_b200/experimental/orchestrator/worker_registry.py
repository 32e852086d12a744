"""Membership table of a run: which workers exist, what they can do, where they sit.

Design. The table is an immutable snapshot (`_Table`) that writers replace as a whole under a
mutex; readers take the current snapshot with one attribute load and never block, so a health
poller, the lifecycle driver's thread pool and a weight-sync round can all walk the membership
while workers come and go. Every change bumps `generation`, which lets a long-running loop notice
cheaply that what it iterated is stale, and is reported to `subscribe`d callbacks (the health
monitor drops state of departed workers that way).

Besides the role index the reference keeps (tunix/experimental/orchestrator/worker_registry.py),
entries are indexed by the GPU rank a worker declares in `WorkerInfo.resources["rank"]`: with
one process per GPU, "the rollout worker on rank 5" is the natural address for peer-memory
weight transfers.

Semantics kept from the reference: ids are unique, a worker must declare at least one role,
`group(role)` of an unknown role is an empty group, listings are sorted by id.
"""
from __future__ import annotations

import dataclasses
import threading
from types import MappingProxyType
from typing import Any, Callable, Dict, Iterator, List, Mapping, Optional, Set, Tuple

from ..common import datatypes
from ..worker import abstract_worker


def _role_key(role: Any) -> str:
  return str(getattr(role, "value", role))


@dataclasses.dataclass(frozen=True)
class _Entry:
  worker: abstract_worker.Worker
  info: datatypes.WorkerInfo
  roles: Tuple[str, ...]
  rank: Optional[int]


@dataclasses.dataclass(frozen=True)
class _Table:
  generation: int = 0
  by_id: Mapping[str, _Entry] = MappingProxyType({})
  by_role: Mapping[str, Tuple[str, ...]] = MappingProxyType({})

  def with_entry(self, e: _Entry) -> "_Table":
    ids = dict(self.by_id)
    ids[e.info.worker_id] = e
    roles = {r: tuple(v) for r, v in self.by_role.items()}
    for r in e.roles:
      roles[r] = roles.get(r, ()) + (e.info.worker_id,)
    return _Table(self.generation + 1, MappingProxyType(ids), MappingProxyType(roles))

  def without(self, worker_id: str) -> "_Table":
    ids = dict(self.by_id)
    gone = ids.pop(worker_id)
    roles = {}
    for r, v in self.by_role.items():
      left = tuple(i for i in v if i != worker_id) if r in gone.roles else v
      if left:
        roles[r] = left
    return _Table(self.generation + 1, MappingProxyType(ids), MappingProxyType(roles))


class WorkerGroup:
  """The workers holding one role at the time the group was taken (a frozen view)."""

  __slots__ = ("role", "_members", "generation")

  def __init__(self, role: str, members: Tuple[abstract_worker.Worker, ...], generation: int = 0):
    self.role, self._members, self.generation = role, tuple(members), generation

  def members(self) -> List[abstract_worker.Worker]:
    return list(self._members)

  def is_empty(self) -> bool:
    return len(self._members) == 0

  def __len__(self) -> int:
    return len(self._members)

  def __iter__(self) -> Iterator[abstract_worker.Worker]:
    return iter(self._members)


class WorkerRegistry:

  def __init__(self):
    self._write = threading.Lock()
    self._table = _Table()
    self._listeners: List[Callable[[str, datatypes.WorkerInfo], None]] = []

  # ---- changes ---------------------------------------------------------------------
  def register(self, worker: abstract_worker.Worker) -> datatypes.WorkerInfo:
    info = worker.info()
    roles = tuple(sorted({_role_key(r) for r in (info.roles or ())}))
    rank = (info.resources or {}).get("rank")
    with self._write:
      if info.worker_id in self._table.by_id:
        raise ValueError(f"duplicate worker_id: {info.worker_id!r}")
      if not roles:
        raise ValueError(f"worker {info.worker_id!r} declares no roles")
      self._table = self._table.with_entry(_Entry(worker, info, roles, None if rank is None else int(rank)))
      listeners = list(self._listeners)
    for fn in listeners:
      fn("registered", info)
    return info

  def unregister(self, worker_id: str) -> None:
    with self._write:
      entry = self._table.by_id.get(worker_id)
      if entry is None:
        raise KeyError(worker_id)
      self._table = self._table.without(worker_id)
      listeners = list(self._listeners)
    for fn in listeners:
      fn("unregistered", entry.info)

  def subscribe(self, fn: Callable[[str, datatypes.WorkerInfo], None]) -> None:
    """`fn(event, info)` runs after every change, event in {"registered", "unregistered"}."""
    with self._write:
      self._listeners.append(fn)

  # ---- lock-free reads of the current snapshot -------------------------------------------
  @property
  def generation(self) -> int:
    return self._table.generation

  def get(self, worker_id: str) -> abstract_worker.Worker:
    return self._table.by_id[worker_id].worker

  def info(self, worker_id: str) -> datatypes.WorkerInfo:
    return self._table.by_id[worker_id].info

  def group(self, role: Any) -> WorkerGroup:
    t, key = self._table, _role_key(role)
    return WorkerGroup(key, tuple(t.by_id[i].worker for i in t.by_role.get(key, ())), t.generation)

  def on_rank(self, rank: int, role: Any = None) -> List[abstract_worker.Worker]:
    """Workers that declared GPU rank `rank` (optionally only those holding `role`)."""
    t, key = self._table, (None if role is None else _role_key(role))
    return [e.worker for _, e in sorted(t.by_id.items()) if e.rank == rank and (key is None or key in e.roles)]

  def roles(self) -> Set[str]:
    return set(self._table.by_role)

  def worker_ids(self) -> List[str]:
    return sorted(self._table.by_id)

  def workers(self) -> List[abstract_worker.Worker]:
    t = self._table
    return [t.by_id[i].worker for i in sorted(t.by_id)]

  def infos(self) -> List[datatypes.WorkerInfo]:
    t = self._table
    return [t.by_id[i].info for i in sorted(t.by_id)]

  def __len__(self) -> int:
    return len(self._table.by_id)

  def __contains__(self, worker_id: str) -> bool:
    return worker_id in self._table.by_id
