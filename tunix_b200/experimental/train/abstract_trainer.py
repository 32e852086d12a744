"""Step-level trainer interface (tunix/experimental/train/abstract_trainer.py:25-191): instead of
owning the loop (`train(dataset)`), the trainer exposes `fwd_bwd` (accumulate gradients of one
micro-batch), `update` (one optimizer step over what was accumulated), `eval_step`, `compile`
(warm-up on dummy data) and checkpoint calls, so an external program decides when each happens."""
from __future__ import annotations

import abc
from typing import Any, Callable, Dict, Optional


class AbstractTrainer(abc.ABC):
  policy_version: int = 0

  @abc.abstractmethod
  def with_loss_fn(self, loss_fn: Callable[..., Any], has_aux: bool = False) -> "AbstractTrainer": ...

  @abc.abstractmethod
  def with_gen_model_input_fn(self, fn: Callable[[Any], Dict[str, Any]]) -> "AbstractTrainer": ...

  @abc.abstractmethod
  def compile(self, dummy_data: Any = None) -> None: ...

  @abc.abstractmethod
  def fwd_bwd(self, payload: Any, **kwargs) -> Any: ...

  @abc.abstractmethod
  def update(self, **kwargs) -> int: ...

  @abc.abstractmethod
  def eval_step(self, payload: Any, **kwargs) -> Any: ...

  def save_checkpoint(self, force: bool = False) -> bool:
    return False

  def restore_checkpoint(self) -> int:
    return 0

  def state_for_weight_sync(self) -> Dict[str, Any]:
    raise NotImplementedError

  def close(self) -> None:
    return None
