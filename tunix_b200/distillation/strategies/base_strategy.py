"""Strategy interface of the distillation trainer (tunix/distillation/strategies/base_strategy.py:38-154)."""
from __future__ import annotations

import abc
from typing import Any, Callable, Dict, Tuple

import torch
import torch.nn.functional as F


def softmax_cross_entropy(logits: torch.Tensor, labels: torch.Tensor) -> torch.Tensor:
  """Per-position cross entropy; `labels` is either a distribution over the last axis
  (one-hot or soft, same shape as logits) or integer class ids (one rank less)."""
  lp = F.log_softmax(logits.float(), dim=-1)
  if labels.dtype in (torch.int32, torch.int64, torch.int16, torch.uint8) and labels.ndim == logits.ndim - 1:
    return -lp.gather(-1, labels.long().unsqueeze(-1)).squeeze(-1)
  return -(labels.to(lp.dtype) * lp).sum(-1)


class BaseStrategy(abc.ABC):
  def __init__(self, student_forward_fn: Callable[..., Any], teacher_forward_fn: Callable[..., Any],
               labels_fn: Callable[..., torch.Tensor]):
    self._student_forward_fn = student_forward_fn
    self._teacher_forward_fn = teacher_forward_fn
    self._labels_fn = labels_fn

  @abc.abstractmethod
  def compute_loss(self, student_output: Any, teacher_output: Any, labels: torch.Tensor): ...

  @abc.abstractmethod
  def compute_eval_loss(self, student_output: Any, labels: torch.Tensor): ...

  def pre_process_models(self, student_model, teacher_model) -> Tuple[Any, Any]:
    return student_model, teacher_model

  def post_process_models(self, student_model, teacher_model) -> Tuple[Any, Any]:
    return student_model, teacher_model

  def get_teacher_outputs(self, teacher_model, inputs: Dict[str, Any]) -> Any:
    with torch.no_grad():
      out = self._teacher_forward_fn(teacher_model, **inputs)
    return out.detach() if isinstance(out, torch.Tensor) else out

  def get_student_outputs(self, student_model, inputs: Dict[str, Any]) -> Any:
    return self._student_forward_fn(student_model, **inputs)

  def get_train_loss(self, student_model, teacher_output: Any, inputs: Dict[str, Any]):
    student_output = self.get_student_outputs(student_model, inputs)
    labels = self._labels_fn(**inputs)
    return self.compute_loss(student_output=student_output, teacher_output=teacher_output, labels=labels)

  def get_eval_loss(self, student_model, inputs: Dict[str, Any]):
    with torch.no_grad():
      student_output = self.get_student_outputs(student_model, inputs)
      labels = self._labels_fn(**inputs)
      return self.compute_eval_loss(student_output=student_output, labels=labels)
