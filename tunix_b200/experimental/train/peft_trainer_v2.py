"""Step-level PEFT trainer on the framework's own training machinery
(role of tunix/experimental/train/peft_trainer_v2.py:60-1486).

It reuses `sft.peft_trainer.PeftTrainer` for everything but the loop: loss / input adapters,
gradient accumulation of unreduced sums divided by the summed denominators at update time,
flat-store optimizer, gradient clipping, metrics logging and checkpoints. `fwd_bwd` runs the
trainer's micro-step without an update, `update` applies the accumulated gradients."""
from __future__ import annotations

from typing import Any, Callable, Dict, List, Optional

import numpy as np
import torch

from ...common.configs import TrainingConfig
from ...common.datatypes import Mode
from ...sft import peft_trainer
from . import abstract_trainer


class PeftTrainerV2(abstract_trainer.AbstractTrainer):
  def __init__(self, model: torch.nn.Module, optimizer, training_config: TrainingConfig):
    self._t = peft_trainer.PeftTrainer(model, optimizer, training_config)
    self._t.is_managed_externally = True
    self._pending = 0
    self._losses: List[float] = []
    self.policy_version = 0

  @property
  def model(self) -> torch.nn.Module:
    return self._t.model

  @property
  def train_steps(self) -> int:
    return self._t.train_steps

  @property
  def metrics_logger(self):
    return self._t.metrics_logger

  def with_loss_fn(self, loss_fn, has_aux: bool = False):
    self._t.with_loss_fn(loss_fn, has_aux)
    return self

  def with_gen_model_input_fn(self, fn):
    self._t.with_gen_model_input_fn(fn)
    return self

  def compile(self, dummy_data: Any = None) -> None:
    """Warm-up: one forward/backward on the dummy batch whose gradients are dropped, so that
    lazy initialisation (kernels, allocator pools, flat stores) happens before serving."""
    if dummy_data is None:
      return
    self._t._train_step(self._t._prepare_inputs(dummy_data), is_update_step=False)
    self._t.grad_accumulator.reset(zero_grads=True)

  def fwd_bwd(self, payload: Any, **kwargs) -> Dict[str, Any]:
    loss, aux, _ = self._t._train_step(self._t._prepare_inputs(payload), is_update_step=False)
    self._pending += 1
    lv = float(loss.detach().float().cpu()) if isinstance(loss, torch.Tensor) else float(loss)
    self._losses.append(lv)
    return {"loss": lv, "pending_micro_batches": self._pending}

  def update(self, **kwargs) -> int:
    if self._pending == 0:
      raise RuntimeError("update() called with no accumulated gradients")
    t = self._t
    if t._grad_sync is not None:
      t._grad_sync.reduce(t.grad_accumulator)
    grad_norm = t._apply_update()
    t._train_steps += 1
    t._log_metrics(float(np.mean(self._losses)), t._train_steps,
                   {"grad_norm": float(grad_norm.detach().float().cpu()) if isinstance(grad_norm, torch.Tensor)
                    else float(grad_norm)})
    self._pending = 0
    self._losses = []
    self.policy_version = t._train_steps
    return t._train_steps

  def eval_step(self, payload: Any, **kwargs) -> Dict[str, Any]:
    with self._t._switch_mode(Mode.EVAL), torch.no_grad():
      loss, _ = self._t._eval_step(self._t._prepare_inputs(payload))
    return {"loss": float(loss.detach().float().cpu()) if isinstance(loss, torch.Tensor) else float(loss)}

  def run_eval(self, eval_ds, **kwargs) -> Dict[str, Any]:
    losses = [self.eval_step(b)["loss"] for b in eval_ds]
    return {"loss": float(np.mean(losses)) if losses else float("nan"), "batches": len(losses)}

  def save_checkpoint(self, force: bool = False) -> bool:
    cm = self._t.checkpoint_manager
    return bool(cm.save(self._t.train_steps, self._t.model, self._t.optimizer, force=force)) if cm else False

  def state_for_weight_sync(self) -> Dict[str, torch.Tensor]:
    lora = any(getattr(p, "is_lora", False) for p in self.model.parameters())
    return {n: p.detach() for n, p in self.model.named_parameters() if getattr(p, "is_lora", False) or not lora}

  def close(self) -> None:
    self._t.close()
