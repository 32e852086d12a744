"""Worker around a step-level trainer (tunix/experimental/worker/trainer_worker.py:30-265): exposes
`fwd_bwd` / `update` / `train_step` / `eval_step` / checkpoints to an orchestrator, keeps the
lifecycle state, and is the SOURCE side of weight-sync rounds."""
from __future__ import annotations

import functools
import inspect
from typing import Any, Callable, Dict, Optional, Sequence

from ..common import datatypes
from ..orchestrator import peer_memory_handler, weight_sync
from ..train import abstract_trainer
from . import abstract_worker

WorkerState = datatypes.WorkerState


def _serving(method):
  """An API call that needs a READY worker (a PENDING one is initialised on the way) and whose failure puts the
  worker into ERROR with the message kept for the next heartbeat."""
  @functools.wraps(method)
  def guarded(self: "TrainerWorker", *args, **kwargs):
    if self.state == WorkerState.PENDING:
      self.initialize()
    if self.state != WorkerState.READY:
      raise RuntimeError(f"TrainerWorker is not ready: {self.state.value}.")
    try:
      result = method(self, *args, **kwargs)
    except Exception as e:
      self._last_error = str(e)
      self._state = WorkerState.ERROR
      raise
    self._last_error = None
    return result
  return guarded


class TrainerWorker(abstract_worker.Worker):
  """Everything a caller learns comes back as a `Response` whose metadata carries the worker id, its state and the
  policy version next to the call's own fields (`_reply`); trainer return values that are dicts are merged in."""

  ROLES = frozenset({"trainer", "actor", "weight_sync"})

  def __init__(self, trainer_factory: Callable[[], abstract_trainer.AbstractTrainer], *,
               worker_id: str = "trainer_worker", handler: Optional[weight_sync.WeightSyncHandler] = None,
               rank: int = 0):
    self._trainer = trainer_factory()
    self._worker_id, self._handler, self._rank = worker_id, handler, rank
    self._state = WorkerState.PENDING
    self._last_error: Optional[str] = None
    self._staged: Optional[Dict[str, Any]] = None

  @property
  def trainer(self) -> abstract_trainer.AbstractTrainer:
    return self._trainer

  @property
  def policy_version(self) -> int:
    return int(getattr(self._trainer, "policy_version", 0))

  def _reply(self, returned: Any = None, **fields) -> datatypes.Response:
    extra = returned if isinstance(returned, dict) else {}
    return datatypes.Response(metadata={"worker_id": self._worker_id, "state": self.state.value,
                                        "policy_version": self.policy_version, **fields, **extra})

  # ---- lifecycle -----------------------------------------------------------------------------
  def initialize(self) -> datatypes.Response:
    if self.state == WorkerState.READY:
      return self._reply(initialized=True, already_ready=True)
    self.state = WorkerState.INITIALIZING
    self.state = WorkerState.READY
    return self._reply(initialized=True)

  def compile(self, dummy_data: Any = None) -> datatypes.Response:
    if self.state == WorkerState.PENDING:
      self.initialize()
    with self._phase(WorkerState.COMPILING):
      try:
        self._trainer.compile(dummy_data)
      except Exception as e:
        self._last_error = str(e)
        raise
    return self._reply(compiled=True)

  def start(self) -> datatypes.Response:
    if self.state == WorkerState.PENDING:
      self.initialize()
    if self.state != WorkerState.READY:
      raise RuntimeError(f"Cannot start TrainerWorker from {self.state.value}.")
    return self._reply(started=True)

  def stop(self) -> datatypes.Response:
    if self.state == WorkerState.STOPPED:
      return self._reply(stopped=True, already_stopped=True)
    if self.state == WorkerState.READY:
      self.state = WorkerState.DRAINING
    try:
      self._trainer.close()
    finally:
      self._state = WorkerState.STOPPED
    return self._reply(stopped=True)

  def info(self) -> datatypes.WorkerInfo:
    return datatypes.WorkerInfo(worker_id=self._worker_id, roles=self.ROLES,
                                resources={"trainer": type(self._trainer).__name__, "policy_version": self.policy_version})

  def heartbeat(self) -> datatypes.HealthReport:
    return datatypes.HealthReport(state=self.state, policy_version=self.policy_version, last_error=self._last_error)

  # ---- configuration -------------------------------------------------------------------------
  def with_loss_fn(self, loss_fn, has_aux: bool = False) -> datatypes.Response:
    self._trainer.with_loss_fn(loss_fn, has_aux)
    return self._reply(loss_fn_configured=True)

  def with_gen_model_input_fn(self, fn) -> datatypes.Response:
    self._trainer.with_gen_model_input_fn(fn)
    return self._reply(gen_model_input_fn_configured=True)

  # ---- training API --------------------------------------------------------------------------
  @_serving
  def fwd_bwd(self, payload: Any, **kwargs) -> datatypes.Response:
    kwargs.pop("skip_jit", None)                 # a tracing-compiler switch of the reference's API; nothing to skip here
    return self._reply(self._trainer.fwd_bwd(payload, **kwargs), queued=True)

  @_serving
  def update(self, **kwargs) -> int:
    return self._trainer.update(**kwargs)

  def train_step(self, payload: Any, accumulate_gradients: bool = False, apply_optimizer: bool = True,
                 **kwargs) -> datatypes.Response:
    """`fwd_bwd` on the payload, then `update` when `apply_optimizer`."""
    reply = self.fwd_bwd(payload, **kwargs)
    if apply_optimizer:
      reply.metadata["train_steps"] = self.update()
      reply.metadata["policy_version"] = self.policy_version
    return reply

  @_serving
  def eval_step(self, payload: Any, **kwargs) -> datatypes.Response:
    return self._reply(self._trainer.eval_step(payload, **kwargs), evaluated=True)

  @_serving
  def run_eval(self, eval_ds: Any, **kwargs) -> datatypes.Response:
    if eval_ds is None:
      return self._reply(evaluated=True, eval_batches=0)
    own = getattr(self._trainer, "run_eval", None)
    if callable(own):
      return self._reply(own(eval_ds, **kwargs), evaluated=True)
    batches = 0
    for batch in eval_ds:
      self._trainer.eval_step(batch)
      batches += 1
    return self._reply(evaluated=True, batches=batches)

  def save_checkpoint(self, force: bool = False) -> datatypes.Response:
    return self._reply(saved=bool(self._trainer.save_checkpoint(force)))

  # ---- weight-sync source --------------------------------------------------------------------
  @property
  def work_unit(self) -> weight_sync.WorkUnitId:
    return weight_sync.WorkUnitId(job_name="trainer", job_replica_id=self._worker_id, data_replica_idx=self._rank)

  async def prepare_weight_sync(self, sync_request: Any = None, **kwargs) -> Sequence[weight_sync.WorkUnitMetadata]:
    """Exposes the current weights to the transport and describes them. The worker is SYNCING from here until
    `release_weight_sync`, so no training call changes the weights under the transfer; a failure leaves it in
    ERROR. A trainer that stages its weights itself (`prepare_weight_sync` of its own) is asked first."""
    if self.state == WorkerState.PENDING:
      self.initialize()
    self.state = WorkerState.SYNCING
    try:
      own = getattr(self._trainer, "prepare_weight_sync", None)
      if callable(own):
        return await _maybe_await(own(sync_request=sync_request, **kwargs))
      self._staged = self._trainer.state_for_weight_sync()
      attach = getattr(self._handler, "attach", None)
      if callable(attach):
        attach(self.work_unit, self._staged)
      return [peer_memory_handler.manifest_of(self.work_unit, self._staged)]
    except Exception as e:
      self._last_error = str(e)
      self._state = WorkerState.ERROR
      raise

  async def release_weight_sync(self, sync_request: Any = None, **kwargs) -> Any:
    """Ends the round on the source: the staged view is dropped, the trainer's own release hook (when it has one)
    runs, and the worker serves training calls again - also when the hook raises, since the round is over."""
    self._staged = None
    try:
      own = getattr(self._trainer, "release_weight_sync", None)
      return await _maybe_await(own(sync_request=sync_request, **kwargs)) if callable(own) else None
    finally:
      if self.state == WorkerState.SYNCING:
        self.state = WorkerState.READY


async def _maybe_await(value: Any) -> Any:
  return await value if inspect.isawaitable(value) else value
