"""Hook interfaces the trainer calls around steps and batches (tunix/sft/hooks.py:25-77)."""
from __future__ import annotations

import abc
from typing import Any


class TrainingHooks(abc.ABC):
  """Callbacks around training / evaluation steps."""

  def on_train_start(self, train_ctx: Any) -> None:
    pass

  def on_train_end(self, train_ctx: Any) -> None:
    pass

  def on_train_step_start(self, train_ctx: Any) -> None:
    pass

  def on_train_step_end(self, train_ctx: Any, train_step: int, train_loss: float) -> None:
    pass

  def on_eval_step_start(self, train_ctx: Any) -> None:
    pass

  def on_eval_step_end(self, train_ctx: Any, eval_loss: float) -> None:
    pass


class DataHooks(abc.ABC):
  """Callbacks that supply batches instead of the dataset iterators."""

  @abc.abstractmethod
  def load_next_train_batch(self, train_ctx: Any) -> Any:
    ...

  @abc.abstractmethod
  def load_next_eval_batch(self, train_ctx: Any) -> Any:
    ...
