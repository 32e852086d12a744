"""Strictly synchronous weight-sync rounds over the worker registry
(tunix/experimental/orchestrator/weight_sync_coordinator.py:15-1558).

One round:  bind + metadata on every destination and prepare on every source (all still
serving) -> register every work unit with the handler -> pre on every destination (downtime
starts: admission closed, drained, KV cache freed) -> handler.transfer -> weight_sync on every
destination (into staging only) -> post on every destination (atomic publish, resume) ->
release on every source.

Failure handling keeps version consistency and worker health apart:
  * a failure before any publish rolls back: every destination that was asked to prepare gets
    `abort_weight_sync`; all confirm -> ABORTED (fleet serves the old version, coordinator stays
    usable); some cannot confirm -> FAILED_NEEDS_RESTART;
  * some destinations published and others did not -> PARTIALLY_COMMITTED;
  * the transfer call timed out or its outcome is unknown -> UNKNOWN_TRANSFER_STATE: nothing is
    aborted and source staging is NOT released, because the transport may still be writing.
After any of the last three the coordinator is poisoned and `sync` raises until
`reset_after_recovery()`.

Publishing is retried: `post_weight_sync` is idempotent on a worker (its tracker ignores a second delivery),
so destinations whose publish failed are asked again (`post_retries` times) before the round is judged. If
after that NO destination has published, the fleet is still uniform and the round is rolled back like any
other pre-publish failure instead of poisoning the coordinator.

Cancellation (the caller's task is cancelled mid-round) never leaves the fleet quiesced: between the start of
the downtime and the publish the destinations are rolled back and the sources released before the
cancellation propagates; a cancellation during the transfer call parks the round as UNKNOWN_TRANSFER_STATE
(nothing touched, coordinator poisoned); one during the publish lets the publish finish on every destination
first, so the fleet converges on the new version or, failing that, is reported PARTIALLY_COMMITTED. The
outcome of a cancelled round is kept in `last_result`.

A failed phase call means "the reply is lost", not "the work did not happen": before deciding,
the coordinator asks the worker for its round report (`get_weight_sync_status`) and accepts the
phase if the report proves it. Workers key their round by the (req_id, uuid) carried in
`WeightSyncRequest.extra_config`; `WorkerRoundTracker` implements the worker side: idempotent
phases, rejection of stale rounds and of mid-round phases for rounds the worker never opened.
"""
from __future__ import annotations

import asyncio
import dataclasses
import enum
import inspect
import logging
import threading
from typing import Any, Dict, List, Optional, Sequence, Tuple

from ..common import datatypes
from . import weight_sync, worker_registry

TRAINER_ROLE = "trainer"
ROLLOUT_ROLE = "rollout"

# worker-reported phases that prove a coordinator call's work happened
_PHASE_ACCEPTS = {
    "pre_weight_sync": frozenset({"prepared", "h2d_done", "committed"}),
    "weight_sync": frozenset({"h2d_done", "committed"}),
    "post_weight_sync": frozenset({"committed"}),
    "abort_weight_sync": frozenset({"aborted"}),
}
_PHASE_ORDER = {"idle": 0, "prepared": 1, "h2d_done": 2, "committed": 3, "aborted": 3}
_ROUND_OPENING_PHASES = frozenset({"prepared", "aborted"})


class StaleRoundError(RuntimeError):
  """A phase call belongs to an older round, reuses a round key, or tries to continue a round
  this worker never opened."""


class WorkerRoundTracker:
  """Worker-side round bookkeeping. Usage inside a phase method:

      if tracker.admit(request, "h2d_done"):
        ...do the (re-runnable) work...
        tracker.complete(request, "h2d_done")

  `admit` -> False for a duplicate delivery (phase already reached), raises `StaleRoundError`
  for stale / foreign keys, opens a new round only for "prepared" or "aborted"."""

  def __init__(self):
    self._lock = threading.Lock()
    self._req_id: Optional[str] = None
    self._uuid = -1
    self._phase = "idle"
    self._policy_version = -1

  @staticmethod
  def _key(req: Any) -> Tuple[str, int]:
    extra = getattr(req, "extra_config", None) or {}
    return extra.get("req_id", ""), int(extra.get("uuid", 0))

  def admit(self, req: Any, phase: str) -> bool:
    rid, uuid = self._key(req)
    with self._lock:
      if self._req_id is not None and uuid < self._uuid:
        raise StaleRoundError(f"phase {phase!r} for round (req_id={rid!r}, uuid={uuid}) rejected: this worker is on "
                              f"uuid {self._uuid}")
      if self._req_id is not None and uuid == self._uuid and rid != self._req_id:
        raise StaleRoundError(f"phase {phase!r} carries uuid {uuid} under req_id {rid!r}, but this worker's round "
                              f"{uuid} is req_id {self._req_id!r}; a round key must never be reused")
      if self._req_id is None or uuid > self._uuid:
        if phase not in _ROUND_OPENING_PHASES:
          raise StaleRoundError(f"phase {phase!r} cannot open a round: (req_id={rid!r}, uuid={uuid}) is unknown to "
                                f"this worker, which is on uuid {self._uuid}; only a pre or an abort may start a round")
        self._req_id, self._uuid, self._phase = rid, uuid, "idle"
        self._policy_version = getattr(req, "policy_version", -1)
      if phase == "committed" and self._phase == "aborted":
        raise StaleRoundError(f"commit refused: round (req_id={rid!r}, uuid={uuid}) was already aborted on this worker")
      if phase == "aborted" and self._phase == "committed":
        return False
      if self._phase != "idle" and _PHASE_ORDER[phase] <= _PHASE_ORDER.get(self._phase, 0):
        return False
      return True

  def complete(self, req: Any, phase: str) -> None:
    rid, uuid = self._key(req)
    with self._lock:
      if uuid != self._uuid or (self._req_id is not None and rid != self._req_id):
        raise StaleRoundError(f"complete({phase!r}) for round (req_id={rid!r}, uuid={uuid}) but the worker is on "
                              f"(req_id={self._req_id!r}, uuid={self._uuid})")
      self._phase = phase
      self._policy_version = getattr(req, "policy_version", self._policy_version)

  def report(self) -> Dict[str, Any]:
    with self._lock:
      return {"req_id": self._req_id, "uuid": self._uuid, "phase": self._phase,
              "policy_version": self._policy_version}


class RoundState(enum.Enum):
  IDLE = "idle"
  PREPARING = "preparing"
  PREPARED = "prepared"
  TRANSFERRING = "transferring"
  H2D_IN_PROGRESS = "h2d_in_progress"
  PENDING_COMMIT = "pending_commit"
  COMMITTED = "committed"
  ABORTED = "aborted"
  PARTIALLY_COMMITTED = "partially_committed"
  FAILED_NEEDS_RESTART = "failed_needs_restart"
  UNKNOWN_TRANSFER_STATE = "unknown_transfer_state"


_POISONING_STATES = frozenset({RoundState.PARTIALLY_COMMITTED, RoundState.FAILED_NEEDS_RESTART,
                               RoundState.UNKNOWN_TRANSFER_STATE})


@dataclasses.dataclass(frozen=True)
class PhaseTimeouts:
  bind: float = 60.0
  metadata: float = 60.0
  source_prepare: float = 900.0
  pre: float = 180.0
  transfer: float = 1800.0
  h2d: float = 900.0
  post: float = 300.0
  abort: float = 180.0
  status: float = 30.0
  release: float = 120.0


@dataclasses.dataclass(frozen=True)
class WorkerRoundReport:
  worker_id: str
  phase: str                   # last self-reported phase; "unknown" when unreachable
  error: str = ""
  needs_restart: bool = False


@dataclasses.dataclass(frozen=True)
class WeightSyncResult:
  policy_version: int
  round_index: int
  req_id: str
  uuid: int
  state: RoundState
  transfer: Optional[weight_sync.TransferResult]
  source_units: Tuple[weight_sync.WorkUnitId, ...]
  destination_units: Tuple[weight_sync.WorkUnitId, ...]
  workers: Tuple[WorkerRoundReport, ...] = ()
  failures: Tuple[str, ...] = ()

  @property
  def success(self) -> bool:
    return self.state == RoundState.COMMITTED


class WeightSyncError(RuntimeError):
  def __init__(self, message: str, result: WeightSyncResult):
    super().__init__(message)
    self.result = result


class Manifest:
  """What one side of a round says it holds: variable name -> (global shape, bytes per element).

  Built from the work-unit metadata of every member of the side. Units of one side describe the same global
  tensors (one unit per host), so two units that disagree about a name are a problem of their own, recorded
  rather than silently overwritten. Multi-tensor units list their variables; a single-tensor unit goes under its
  `data_name`."""

  def __init__(self, side: str, metadata: Sequence[weight_sync.WorkUnitMetadata]):
    self.side = side
    self.entries: Dict[str, Tuple[Optional[Tuple[int, ...]], Optional[int]]] = {}
    self.problems: List[str] = []
    for md in metadata:
      if md.variables:
        for var in md.variables:
          self._add(var.name, tuple(var.shape), var.item_size)
      else:
        self._add(md.unit.data_name, tuple(md.global_shape) if md.global_shape else None, md.item_size)

  def _add(self, name: str, shape, item_size) -> None:
    seen = self.entries.get(name)
    if seen is not None and seen != (shape, item_size):
      self.problems.append(f"preflight: {self.side} units disagree on {name!r}: {seen} vs {(shape, item_size)}")
    self.entries[name] = (shape, item_size)

  def differences(self, other: "Manifest") -> List[str]:
    """Everything that would make a transfer between the two sides lose or corrupt a tensor. The transport pairs
    variables by exact name, so a misspelt name does not fail - it just is not copied; this check costs one
    comparison and runs before any destination stops serving."""
    out = list(self.problems) + list(other.problems)
    mine, theirs = set(self.entries), set(other.entries)
    out += [f"preflight: {self.side} variable {n!r} has no {other.side} counterpart" for n in sorted(mine - theirs)]
    out += [f"preflight: {other.side} variable {n!r} has no {self.side} counterpart" for n in sorted(theirs - mine)]
    for n in sorted(mine & theirs):
      (s_shape, s_item), (d_shape, d_item) = self.entries[n], other.entries[n]
      if s_shape != d_shape:
        out.append(f"preflight: {n!r} global shape differs: {self.side} {s_shape}, {other.side} {d_shape}")
      if s_item != d_item:
        out.append(f"preflight: {n!r} item_size differs: {self.side} {s_item}, {other.side} {d_item}")
    return out


def _worker_id(member: Any) -> str:
  try:
    info = member.info()
    if inspect.isawaitable(info):
      info.close()
      raise TypeError
    return info.worker_id
  except Exception:
    return getattr(member, "worker_id", None) or f"{type(member).__name__}@{id(member):x}"


async def _call(obj: Any, name: str, *args, timeout: Optional[float] = None):
  """Calls a sync or async method with a deadline (sync bodies run on the executor)."""
  fn = getattr(obj, name)
  if inspect.iscoroutinefunction(fn):
    coro = fn(*args)
  else:
    coro = asyncio.get_running_loop().run_in_executor(None, lambda: fn(*args))
  return await asyncio.wait_for(coro, timeout=timeout)


class WeightSyncCoordinator:
  """Drives rounds between the `trainer` role (sources) and the `rollout` role (destinations) of
  a `WorkerRegistry`, or explicit lists of them, through one `WeightSyncHandler`."""

  def __init__(self, handler: weight_sync.WeightSyncHandler, registry: Optional[worker_registry.WorkerRegistry] = None,
               *, sources: Optional[Sequence[Any]] = None, destinations: Optional[Sequence[Any]] = None,
               timeouts: PhaseTimeouts = PhaseTimeouts(), source_role: str = TRAINER_ROLE,
               destination_role: str = ROLLOUT_ROLE, post_retries: int = 1):
    self._handler, self._registry = handler, registry
    self._post_retries = max(0, int(post_retries))
    self.last_result: Optional[WeightSyncResult] = None
    self._explicit_sources, self._explicit_destinations = sources, destinations
    self._timeouts = timeouts
    self._source_role, self._destination_role = source_role, destination_role
    self._round_index = 0
    self._last_committed: Optional[int] = None
    self._poisoned: Optional[str] = None
    self._lock = asyncio.Lock()

  @property
  def round_index(self) -> int:
    return self._round_index

  @property
  def last_committed_version(self) -> Optional[int]:
    return self._last_committed

  @property
  def poisoned(self) -> Optional[str]:
    return self._poisoned

  def reset_after_recovery(self) -> None:
    """To be called once an operator (or a supervisor) has restarted / re-imaged the workers a
    poisoning round left in an unknown state."""
    self._poisoned = None

  def _members(self, role: str, explicit) -> List[Any]:
    if explicit is not None:
      return list(explicit)
    if self._registry is None:
      return []
    return self._registry.group(role).members()

  def _sources(self) -> List[Any]:
    out = self._members(self._source_role, self._explicit_sources)
    if not out:
      raise ValueError(f"no weight-sync source: role {self._source_role!r} has no workers")
    return out

  def _destinations(self) -> List[Any]:
    out = self._members(self._destination_role, self._explicit_destinations)
    if not out:
      raise ValueError(f"no weight-sync destination: role {self._destination_role!r} has no workers")
    return out

  def build_request(self, policy_version: int) -> datatypes.WeightSyncRequest:
    uuid = self._round_index + 1
    req_id = f"weight_sync_v{policy_version}_r{uuid}"
    return datatypes.WeightSyncRequest(request_id=req_id, policy_version=policy_version,
                                       extra_config={"req_id": req_id, "uuid": uuid})

  # ---- phase plumbing ------------------------------------------------------------------------
  async def _phase(self, dest: Any, name: str, req: Any, timeout: float) -> Optional[str]:
    """Runs one destination phase. -> None on success, else an error string. A failed call is
    reconciled against the worker's own round report before it counts as a failure."""
    try:
      await _call(dest, name, req, timeout=timeout)
      return None
    except Exception as e:
      err = f"{name} failed on {_worker_id(dest)}: {type(e).__name__}: {e}"
    try:
      rep = await _call(dest, "get_weight_sync_status", timeout=self._timeouts.status)
      extra = req.extra_config
      if (isinstance(rep, dict) and rep.get("uuid") == extra["uuid"] and rep.get("req_id") == extra["req_id"]
          and rep.get("phase") in _PHASE_ACCEPTS[name]):
        logging.warning("%s; the worker reports phase %r for this round, accepting", err, rep.get("phase"))
        return None
    except Exception:
      pass
    return err

  async def _on_all(self, dests: Sequence[Any], name: str, req: Any, timeout: float) -> Dict[int, Optional[str]]:
    results = await asyncio.gather(*[self._phase(d, name, req, timeout) for d in dests])
    return dict(enumerate(results))

  async def _status(self, dest: Any) -> str:
    try:
      rep = await _call(dest, "get_weight_sync_status", timeout=self._timeouts.status)
      return rep.get("phase", "unknown") if isinstance(rep, dict) else "unknown"
    except Exception:
      return "unknown"

  async def _release(self, sources: Sequence[Any], req: Any) -> List[str]:
    errs = []
    for s in sources:
      try:
        await _call(s, "release_weight_sync", req, timeout=self._timeouts.release)
      except Exception as e:
        errs.append(f"release_weight_sync failed on {_worker_id(s)}: {e}")
    return errs

  async def _rollback(self, dests: Sequence[Any], req: Any) -> Tuple[RoundState, List[WorkerRoundReport], List[str]]:
    errs = await self._on_all(dests, "abort_weight_sync", req, self._timeouts.abort)
    reports, failures = [], []
    for i, d in enumerate(dests):
      if errs[i] is None:
        reports.append(WorkerRoundReport(worker_id=_worker_id(d), phase="aborted"))
      else:
        failures.append(errs[i])
        reports.append(WorkerRoundReport(worker_id=_worker_id(d), phase=await self._status(d), error=errs[i],
                                         needs_restart=True))
    state = RoundState.ABORTED if not failures else RoundState.FAILED_NEEDS_RESTART
    return state, reports, failures

  # ---- a round -------------------------------------------------------------------------------
  async def sync(self, policy_version: int, raise_on_failure: bool = True) -> WeightSyncResult:
    if self._poisoned:
      raise RuntimeError(f"weight-sync coordinator is poisoned by an earlier round ({self._poisoned}); recover the "
                         "workers and call reset_after_recovery()")
    if self._last_committed is not None and policy_version <= self._last_committed:
      raise ValueError(f"policy_version {policy_version} does not advance past the committed version "
                       f"{self._last_committed}")
    async with self._lock:
      result = await self._run_round(policy_version)
    self._record(result)
    if result.state != RoundState.COMMITTED and raise_on_failure:
      raise WeightSyncError(f"weight sync round {result.round_index} ended {result.state.value}: "
                            + "; ".join(result.failures), result)
    return result

  def _record(self, result: WeightSyncResult) -> None:
    self.last_result = result
    if result.state in _POISONING_STATES:
      self._poisoned = f"round {result.round_index} ended {result.state.value}"
    if result.state == RoundState.COMMITTED:
      self._last_committed = result.policy_version

  async def _run_round(self, policy_version: int) -> WeightSyncResult:
    sources, dests = self._sources(), self._destinations()
    req = self.build_request(policy_version)
    self._round_index += 1
    t = self._timeouts
    src_units: List[weight_sync.WorkUnitId] = []
    dst_units: List[weight_sync.WorkUnitId] = []
    transfer: Optional[weight_sync.TransferResult] = None

    def result(state, workers=(), failures=()):
      return WeightSyncResult(policy_version=policy_version, round_index=self._round_index, req_id=req.request_id,
                              uuid=req.extra_config["uuid"], state=state, transfer=transfer,
                              source_units=tuple(src_units), destination_units=tuple(dst_units),
                              workers=tuple(workers), failures=tuple(failures))

    # 1. everything that can happen while both sides still serve
    prepared_sources: List[Any] = []
    try:
      for d in dests:
        await _call(d, "bind_weight_sync", timeout=t.bind)
      dst_meta = [m for d in dests for m in await _call(d, "get_weight_sync_metadata", timeout=t.metadata)]
      src_meta = []
      for s in sources:
        prepared_sources.append(s)
        src_meta += list(await _call(s, "prepare_weight_sync", req, timeout=t.source_prepare))
      mismatches = Manifest("source", src_meta).differences(Manifest("destination", dst_meta))
      if mismatches:
        raise ValueError("; ".join(mismatches[:8]) + (f" (+{len(mismatches) - 8} more)" if len(mismatches) > 8 else ""))
      for m in src_meta + dst_meta:
        self._handler.register_work_unit(m)
      src_units[:] = [m.unit for m in src_meta]
      dst_units[:] = [m.unit for m in dst_meta]
    except Exception as e:
      # nothing is quiesced yet: no rollback needed, just drop the source staging
      failures = [f"preparation failed: {type(e).__name__}: {e}"] + await self._release(prepared_sources, req)
      return result(RoundState.ABORTED, failures=failures)

    # 2..5: the downtime. `stage` tells the cancellation handler what may have happened so far.
    stage = "quiesce"
    try:
      errs = await self._on_all(dests, "pre_weight_sync", req, t.pre)
      if any(errs.values()):
        state, reports, fails = await self._rollback(dests, req)
        fails = [e for e in errs.values() if e] + fails + await self._release(sources, req)
        return result(state, reports, fails)

      stage = "transfer"
      try:
        transfer = await asyncio.wait_for(asyncio.get_running_loop().run_in_executor(
            None, lambda: self._handler.transfer(src_units, dst_units, req_id=req.request_id,
                                                 generation=req.extra_config["uuid"])), timeout=t.transfer)
      except (asyncio.TimeoutError, weight_sync.TransferOutcomeUnknownError) as e:
        # the transport may still be writing: abort nothing, release nothing
        return result(RoundState.UNKNOWN_TRANSFER_STATE, await self._parked(dests),
                      [f"transfer outcome unknown: {type(e).__name__}: {e}"])
      except asyncio.CancelledError:
        raise
      except Exception as e:
        transfer = weight_sync.TransferResult(req_id=req.request_id, success=False, message=f"{type(e).__name__}: {e}")
      stage = "stage"
      if not transfer.success:
        state, reports, fails = await self._rollback(dests, req)
        fails = [f"transfer failed: {transfer.message}"] + fails + await self._release(sources, req)
        return result(state, reports, fails)

      errs = await self._on_all(dests, "weight_sync", req, t.h2d)
      if any(errs.values()):
        state, reports, fails = await self._rollback(dests, req)
        fails = [e for e in errs.values() if e] + fails + await self._release(sources, req)
        return result(state, reports, fails)

      stage = "publish"
      return await self._publish(sources, dests, req, result)
    except asyncio.CancelledError:
      outcome = await asyncio.shield(self._settle_cancelled(stage, sources, dests, req, result))
      self._record(outcome)
      raise

  async def _parked(self, dests: Sequence[Any]) -> List[WorkerRoundReport]:
    return [WorkerRoundReport(worker_id=_worker_id(d), phase=await self._status(d), needs_restart=True) for d in dests]

  async def _publish(self, sources, dests, req, result) -> WeightSyncResult:
    """`post_weight_sync` everywhere, retried where it failed; then the verdict."""
    t = self._timeouts
    errs = await self._on_all(dests, "post_weight_sync", req, t.post)
    for _ in range(self._post_retries):
      again = [i for i, e in errs.items() if e]
      if not again:
        break
      retried = await self._on_all([dests[i] for i in again], "post_weight_sync", req, t.post)
      for slot, i in enumerate(again):
        errs[i] = retried[slot]
    failed = [i for i, e in errs.items() if e]
    if not failed:
      release_errs = await self._release(sources, req)
      reports = [WorkerRoundReport(worker_id=_worker_id(d), phase="committed") for d in dests]
      return result(RoundState.COMMITTED, reports, release_errs)
    phases = {i: ("committed" if errs[i] is None else await self._status(dests[i])) for i in range(len(dests))}
    if "committed" not in phases.values() and "unknown" not in phases.values():
      # nobody published and everybody answers: the fleet is uniform on the old version, so roll back
      state, reports, fails = await self._rollback(dests, req)
      fails = [errs[i] for i in failed] + fails + await self._release(sources, req)
      return result(state, reports, fails)
    release_errs = await self._release(sources, req)
    reports = [WorkerRoundReport(worker_id=_worker_id(d), phase=phases[i], error=errs[i] or "",
                                 needs_restart=errs[i] is not None) for i, d in enumerate(dests)]
    committed = sum(1 for r in reports if r.phase == "committed")
    state = RoundState.PARTIALLY_COMMITTED if committed else RoundState.FAILED_NEEDS_RESTART
    return result(state, reports, [errs[i] for i in failed] + release_errs)

  async def _settle_cancelled(self, stage: str, sources, dests, req, result) -> WeightSyncResult:
    """Brings a round whose driver was cancelled to a defined end (runs shielded from further cancellation)."""
    note = f"round cancelled during {stage}"
    if stage == "transfer":
      return result(RoundState.UNKNOWN_TRANSFER_STATE, await self._parked(dests), [note])
    if stage == "publish":
      outcome = await self._publish(sources, dests, req, result)
      return dataclasses.replace(outcome, failures=(note,) + tuple(outcome.failures))
    state, reports, fails = await self._rollback(dests, req)
    return result(state, reports, [note] + fails + await self._release(sources, req))
