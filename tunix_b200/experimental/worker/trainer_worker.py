"""Worker around a step-level trainer (tunix/experimental/worker/trainer_worker.py:30-265): exposes
`fwd_bwd` / `update` / `train_step` / `eval_step` / checkpoints to an orchestrator, keeps the
lifecycle state, and is the SOURCE side of weight-sync rounds."""
from __future__ import annotations

from typing import Any, Callable, Dict, Optional, Sequence

from ..common import datatypes
from ..orchestrator import peer_memory_handler, weight_sync
from ..train import abstract_trainer
from . import abstract_worker

WorkerState = datatypes.WorkerState


class TrainerWorker(abstract_worker.Worker):
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

  def _version(self) -> int:
    return int(getattr(self._trainer, "policy_version", 0))

  def _response(self, **md) -> datatypes.Response:
    return datatypes.Response(metadata={"worker_id": self._worker_id, "state": self.state.value,
                                        "policy_version": self._version(), **md})

  def _ensure_ready(self) -> None:
    if self.state == WorkerState.PENDING:
      self.initialize()
    if self.state != WorkerState.READY:
      raise RuntimeError(f"TrainerWorker is not ready: {self.state.value}.")

  def _guard(self, fn, *a, **k):
    try:
      out = fn(*a, **k)
      self._last_error = None
      return out
    except Exception as e:
      self._last_error = str(e)
      self._state = WorkerState.ERROR
      raise

  # ---- lifecycle -----------------------------------------------------------------------------
  def initialize(self) -> datatypes.Response:
    if self.state == WorkerState.READY:
      return self._response(initialized=True, already_ready=True)
    self.state = WorkerState.INITIALIZING
    self.state = WorkerState.READY
    return self._response(initialized=True)

  def compile(self, dummy_data: Any = None) -> datatypes.Response:
    if self.state == WorkerState.PENDING:
      self.initialize()
    with self._phase(WorkerState.COMPILING):
      self._guard(self._trainer.compile, dummy_data)
    return self._response(compiled=True)

  def start(self) -> datatypes.Response:
    if self.state == WorkerState.PENDING:
      self.initialize()
    if self.state != WorkerState.READY:
      raise RuntimeError(f"Cannot start TrainerWorker from {self.state.value}.")
    return self._response(started=True)

  def stop(self) -> datatypes.Response:
    if self.state == WorkerState.STOPPED:
      return self._response(stopped=True, already_stopped=True)
    if self.state == WorkerState.READY:
      self.state = WorkerState.DRAINING
    try:
      self._trainer.close()
    finally:
      self._state = WorkerState.STOPPED
    return self._response(stopped=True)

  def info(self) -> datatypes.WorkerInfo:
    return datatypes.WorkerInfo(worker_id=self._worker_id, roles=frozenset({"trainer", "actor", "weight_sync"}),
                                resources={"trainer": type(self._trainer).__name__, "policy_version": self._version()})

  def heartbeat(self) -> datatypes.HealthReport:
    return datatypes.HealthReport(state=self.state, policy_version=self._version(), last_error=self._last_error)

  # ---- training API --------------------------------------------------------------------------
  def with_loss_fn(self, loss_fn, has_aux: bool = False) -> datatypes.Response:
    self._trainer.with_loss_fn(loss_fn, has_aux)
    return self._response(loss_fn_configured=True)

  def with_gen_model_input_fn(self, fn) -> datatypes.Response:
    self._trainer.with_gen_model_input_fn(fn)
    return self._response(gen_model_input_fn_configured=True)

  def fwd_bwd(self, payload: Any, **kwargs) -> datatypes.Response:
    self._ensure_ready()
    kwargs.pop("skip_jit", None)
    out = self._guard(self._trainer.fwd_bwd, payload, **kwargs)
    return self._response(queued=True, **(out if isinstance(out, dict) else {}))

  def update(self, **kwargs) -> int:
    self._ensure_ready()
    return self._guard(self._trainer.update, **kwargs)

  def train_step(self, payload: Any, accumulate_gradients: bool = False, apply_optimizer: bool = True,
                 **kwargs) -> datatypes.Response:
    """`fwd_bwd` on the payload, then `update` when `apply_optimizer`."""
    r = self.fwd_bwd(payload, **kwargs)
    if apply_optimizer:
      r.metadata["train_steps"] = self.update()
      r.metadata["policy_version"] = self._version()
    return r

  def eval_step(self, payload: Any, **kwargs) -> datatypes.Response:
    self._ensure_ready()
    out = self._guard(self._trainer.eval_step, payload, **kwargs)
    return self._response(evaluated=True, **(out if isinstance(out, dict) else {}))

  def run_eval(self, eval_ds: Any, **kwargs) -> datatypes.Response:
    self._ensure_ready()
    if eval_ds is None:
      return self._response(evaluated=True, eval_batches=0)
    fn = getattr(self._trainer, "run_eval", None)
    out = self._guard(fn, eval_ds, **kwargs) if callable(fn) else {"batches": sum(1 for b in eval_ds
                                                                                  if self._trainer.eval_step(b) or True)}
    return self._response(evaluated=True, **(out if isinstance(out, dict) else {}))

  def save_checkpoint(self, force: bool = False) -> datatypes.Response:
    return self._response(saved=bool(self._trainer.save_checkpoint(force)))

  # ---- weight-sync source --------------------------------------------------------------------
  @property
  def work_unit(self) -> weight_sync.WorkUnitId:
    return weight_sync.WorkUnitId(job_name="trainer", job_replica_id=self._worker_id, data_replica_idx=self._rank)

  async def prepare_weight_sync(self, sync_request: Any = None, **kwargs) -> Sequence[weight_sync.WorkUnitMetadata]:
    state = self._trainer.state_for_weight_sync()
    self._staged = state
    if self._handler is not None and hasattr(self._handler, "attach"):
      self._handler.attach(self.work_unit, state)
    return [peer_memory_handler.manifest_of(self.work_unit, state)]

  async def release_weight_sync(self, sync_request: Any = None, **kwargs) -> None:
    self._staged = None
