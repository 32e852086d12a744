"""Registry of live workers by id and by role (tunix/experimental/orchestrator/worker_registry.py:29-145).
Registration snapshots the worker's `WorkerInfo`; all accessors are thread-safe and return
copies, so a poller can iterate while another thread registers or removes workers."""
from __future__ import annotations

import threading
from typing import Dict, Iterator, List, Set

from ..common import datatypes
from ..worker import abstract_worker


class WorkerGroup:
  def __init__(self, role: str, members: List[abstract_worker.Worker]):
    self._role, self._members = role, list(members)

  @property
  def role(self) -> str:
    return self._role

  def members(self) -> List[abstract_worker.Worker]:
    return list(self._members)

  def is_empty(self) -> bool:
    return not self._members

  def __len__(self) -> int:
    return len(self._members)

  def __iter__(self) -> Iterator[abstract_worker.Worker]:
    return iter(self._members)


class WorkerRegistry:
  def __init__(self):
    self._lock = threading.RLock()
    self._workers: Dict[str, abstract_worker.Worker] = {}
    self._infos: Dict[str, datatypes.WorkerInfo] = {}
    self._role_to_ids: Dict[str, List[str]] = {}

  def register(self, worker: abstract_worker.Worker) -> datatypes.WorkerInfo:
    info = worker.info()
    with self._lock:
      if info.worker_id in self._workers:
        raise ValueError(f"duplicate worker_id: {info.worker_id!r}")
      if not info.roles:
        raise ValueError(f"worker {info.worker_id!r} declares no roles")
      self._workers[info.worker_id] = worker
      self._infos[info.worker_id] = info
      for role in info.roles:
        self._role_to_ids.setdefault(str(getattr(role, "value", role)), []).append(info.worker_id)
    return info

  def unregister(self, worker_id: str) -> None:
    with self._lock:
      if worker_id not in self._workers:
        raise KeyError(worker_id)
      info = self._infos.pop(worker_id)
      del self._workers[worker_id]
      for role in info.roles:
        key = str(getattr(role, "value", role))
        self._role_to_ids[key].remove(worker_id)
        if not self._role_to_ids[key]:
          del self._role_to_ids[key]

  def get(self, worker_id: str) -> abstract_worker.Worker:
    with self._lock:
      return self._workers[worker_id]

  def info(self, worker_id: str) -> datatypes.WorkerInfo:
    with self._lock:
      return self._infos[worker_id]

  def group(self, role) -> WorkerGroup:
    key = str(getattr(role, "value", role))
    with self._lock:
      return WorkerGroup(key, [self._workers[i] for i in self._role_to_ids.get(key, [])])

  def roles(self) -> Set[str]:
    with self._lock:
      return set(self._role_to_ids)

  def worker_ids(self) -> List[str]:
    with self._lock:
      return sorted(self._workers)

  def workers(self) -> List[abstract_worker.Worker]:
    with self._lock:
      return [self._workers[i] for i in sorted(self._workers)]

  def infos(self) -> List[datatypes.WorkerInfo]:
    with self._lock:
      return [self._infos[i] for i in sorted(self._workers)]

  def __len__(self) -> int:
    with self._lock:
      return len(self._workers)

  def __contains__(self, worker_id: str) -> bool:
    with self._lock:
      return worker_id in self._workers
