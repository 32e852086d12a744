"""Cluster supervisor (tunix/experimental/orchestrator/orchestrator.py:41-288): owns the worker
registry (local workers) and remote worker handles, brings everything up phase by phase,
validates the run geometry, builds the `DistributedRLEngine` over the role groups, runs an RL
program on it, polls health, and shuts down best-effort."""
from __future__ import annotations

import collections
import logging
from concurrent import futures
from typing import Any, Dict, List, Optional, Sequence

from ..common import datatypes
from ..worker import abstract_worker, remote_execution
from . import distributed_rl_engine, health_monitor, lifecycle, rl_program, startup_validation, worker_registry

_STOP_TIMEOUT_S = 60.0


def _role_key(role) -> str:
  return str(getattr(role, "value", role)).lower()


class ClusterOrchestrator:
  def __init__(self, config: Any = None, registry: Optional[worker_registry.WorkerRegistry] = None,
               lifecycle_driver: Optional[lifecycle.LifecycleDriver] = None,
               monitor: Optional[health_monitor.HealthMonitor] = None, weight_sync_coordinator: Any = None):
    self.config = config
    self.registry = registry or worker_registry.WorkerRegistry()
    self.lifecycle_driver = lifecycle_driver or lifecycle.LifecycleDriver(self.registry)
    self.monitor = monitor or health_monitor.HealthMonitor(self.registry)
    self._remote_by_role: Dict[str, List[remote_execution.ActorHandle]] = collections.defaultdict(list)
    self._remote_by_id: Dict[str, remote_execution.ActorHandle] = {}
    self._remote_infos: Dict[str, datatypes.WorkerInfo] = {}
    self.engine: Optional[distributed_rl_engine.DistributedRLEngine] = None
    self._weight_sync_coordinator = weight_sync_coordinator

  def __enter__(self) -> "ClusterOrchestrator":
    self.bring_up_workers()
    return self

  def __exit__(self, *exc) -> None:
    self.shutdown()

  # ---- registration --------------------------------------------------------------------------
  def register_worker(self, worker: abstract_worker.Worker) -> datatypes.WorkerInfo:
    if worker.info().worker_id in self._remote_infos:
      raise ValueError(f"duplicate worker_id: {worker.info().worker_id!r}")
    return self.registry.register(worker)

  def register_worker_handle(self, worker_id: str, roles: Sequence[Any], handle: remote_execution.ActorHandle,
                             resources: Optional[Dict[str, Any]] = None) -> datatypes.WorkerInfo:
    if not roles:
      raise ValueError(f"worker {worker_id!r} declares no roles")
    if not isinstance(handle, remote_execution.ActorHandle):
      raise TypeError(f"register_worker_handle expects a remote_execution.ActorHandle, got {type(handle)}")
    if worker_id in self._remote_infos or worker_id in self.registry:
      raise ValueError(f"duplicate worker_id: {worker_id!r}")
    names = frozenset(_role_key(r) for r in roles)
    info = datatypes.WorkerInfo(worker_id=worker_id, roles=names, resources={"remote": True, **(resources or {})})
    for r in names:
      self._remote_by_role[r].append(handle)
    self._remote_by_id[worker_id] = handle
    self._remote_infos[worker_id] = info
    return info

  def unregister_worker(self, worker_id: str) -> None:
    if worker_id in self._remote_infos:
      info, handle = self._remote_infos.pop(worker_id), self._remote_by_id.pop(worker_id)
      for r in info.roles:
        self._remote_by_role[r] = [h for h in self._remote_by_role.get(r, []) if h is not handle]
        if not self._remote_by_role[r]:
          del self._remote_by_role[r]
      return
    self.registry.unregister(worker_id)

  def worker_infos(self) -> List[datatypes.WorkerInfo]:
    return self.registry.infos() + [self._remote_infos[i] for i in sorted(self._remote_infos)]

  # ---- lifecycle -----------------------------------------------------------------------------
  def bring_up_workers(self, dummy_data: Any = None) -> None:
    self.lifecycle_driver.bring_up(dummy_data)
    ids = sorted(self._remote_infos)
    for phase, args in (("initialize", ()), ("compile", (dummy_data,)), ("start", ())):
      failures = []
      for wid in ids:
        try:
          self._remote_by_id[wid].submit(phase, *args)
        except Exception as e:
          failures.append((wid, e))
      if failures:
        raise lifecycle.LifecycleError(phase, failures)
    self.engine = self._create_engine()

  def shutdown(self) -> None:
    self.monitor.close()
    pool = futures.ThreadPoolExecutor(max_workers=4)
    stops = {wid: pool.submit(self._remote_by_id[wid].submit, "stop") for wid in sorted(self._remote_infos)}
    for wid, f in stops.items():
      try:
        f.result(timeout=_STOP_TIMEOUT_S)
      except Exception as e:
        logging.warning("Failed to stop remote worker %s: %r", wid, e)
    pool.shutdown(wait=False)
    self.lifecycle_driver.shutdown()

  def validate_startup(self, alg_config: Any, training_config: Any, validators=None) -> None:
    kw = {"validators": validators} if validators is not None else {}
    startup_validation.validate_startup(self.registry, alg_config, training_config, **kw)

  def poll_health(self):
    """-> (reports, overdue workers, unhealthy worker ids) for the local workers."""
    reports = self.monitor.poll()
    return reports, self.monitor.overdue(), self.monitor.unhealthy()

  # ---- engine --------------------------------------------------------------------------------
  def _get_actor_handles(self, role) -> List[remote_execution.ActorHandle]:
    key = _role_key(role)
    handles = list(self._remote_by_role.get(key, ()))
    handles += [remote_execution.InProcessActorHandle(remote_execution.InProcessRemoteExecutionServer(w))
                for w in self.registry.group(key).members()]
    return handles

  def _create_engine(self) -> distributed_rl_engine.DistributedRLEngine:
    R = datatypes.Role
    trainers, inference = {}, {}
    for role in (R.ACTOR, R.CRITIC):
      hs = self._get_actor_handles(role)
      if hs:
        trainers[role] = hs[0]
    for role in (R.REFERENCE, R.REWARD):
      hs = self._get_actor_handles(role)
      if hs:
        inference[role] = hs[0]
    return distributed_rl_engine.DistributedRLEngine(
        rollout_workers=self._get_actor_handles(R.ROLLOUT), trainer_workers=trainers, inference_workers=inference,
        weight_sync_coordinator=self._weight_sync_coordinator)

  def run_program(self, program: rl_program.RLProgram, train_dataset=None, num_steps: Optional[int] = None, **kw):
    if self.engine is None:
      raise RuntimeError("bring_up_workers() must run before a program")
    return program.run(self.engine, train_dataset, num_steps, **kw)

  def run(self, algo: Any, dataset: Any, reward_fns: Optional[Sequence[Any]] = None, assembler: Any = None,
          num_steps: Optional[int] = None, **program_kwargs: Any) -> rl_program.StandardRLProgram:
    """The managed run: brings the workers up if nobody has yet, builds a `StandardRLProgram` from the algorithm
    adapter, the reward functions and the assembler, runs it for `num_steps`, and returns the program (its
    `history` holds one record per step). Weight sync is part of the program only when this orchestrator was given
    a coordinator."""
    if self.engine is None:
      self.bring_up_workers()
    program_kwargs.setdefault("sync_weights", self._weight_sync_coordinator is not None)
    program = rl_program.StandardRLProgram(algo, reward_fns=reward_fns, assembler=assembler, **program_kwargs)
    self.run_program(program, dataset, num_steps=num_steps)
    return program
