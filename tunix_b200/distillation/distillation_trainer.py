"""Distillation trainer: PeftTrainer whose loss is delegated to a strategy.

Behaviour of tunix/distillation/distillation_trainer.py:40-170: the strategy may wrap both
models before training (feature capture, projection head) and unwraps them in `close()`;
teacher outputs are computed once per batch in `_prepare_inputs` (train mode only, without
gradients); strategies return a scalar loss or `(loss, metrics)` and the metrics are logged.
"""
from __future__ import annotations

import dataclasses
from typing import Any, Callable, Dict, Tuple

import numpy as np
import torch

from ..common.configs import TrainingConfig
from ..common.datatypes import Mode
from ..sft import peft_trainer
from . import strategies


@dataclasses.dataclass
class TrainingInput(peft_trainer.TrainingInput):
  teacher_output: Any = None


class DistillationTrainer(peft_trainer.PeftTrainer):
  def __init__(self, student_model: torch.nn.Module, teacher_model: torch.nn.Module,
               strategy: strategies.BaseStrategy, optimizer, training_config: TrainingConfig):
    student_model, teacher_model = strategy.pre_process_models(student_model, teacher_model)
    super().__init__(student_model, optimizer, training_config)
    self.strategy = strategy
    self.teacher_model = teacher_model
    self.teacher_model.eval()
    self.loss_fn = self.get_train_loss
    self.eval_loss_fn = self.get_eval_loss
    self._has_aux = True
    self._seen_metrics: Dict[str, Callable] = {}
    self.gen_model_input_fn = lambda x: {
        "inputs": {"input_tokens": x.input_tokens, "input_mask": x.input_mask},
        "teacher_output": getattr(x, "teacher_output", None)}

  def with_gen_model_input_fn(self, gen_model_input_fn):
    self.gen_model_input_fn = lambda x: {"inputs": gen_model_input_fn(x),
                                         "teacher_output": getattr(x, "teacher_output", None)}
    return self

  def with_loss_fn(self, loss_fn, has_aux: bool = False):
    raise NotImplementedError("with_loss_fn is not supported for distillation. Use the strategy to define the loss.")

  def _to_device(self, v):
    if isinstance(v, np.ndarray):
      v = torch.from_numpy(v)
    return v.to(self._device) if isinstance(v, torch.Tensor) else v

  def _prepare_inputs(self, input_data: Any) -> TrainingInput:
    input_data = dataclasses.replace(input_data, input_tokens=self._to_device(input_data.input_tokens),
                                     input_mask=self._to_device(input_data.input_mask)) \
        if dataclasses.is_dataclass(input_data) else input_data
    inputs = self.gen_model_input_fn(input_data)["inputs"]
    teacher_output = None
    if self._mode != Mode.EVAL:
      teacher_output = self.strategy.get_teacher_outputs(self.teacher_model, inputs)
    return TrainingInput(input_tokens=input_data.input_tokens, input_mask=input_data.input_mask,
                         images=getattr(input_data, "images", None), teacher_output=teacher_output)

  @staticmethod
  def _standardize_loss_output(output: Any) -> Tuple[Any, Dict[str, Any]]:
    return output if isinstance(output, tuple) else (output, {})

  def get_train_loss(self, model, teacher_output, inputs):
    return self._standardize_loss_output(self.strategy.get_train_loss(model, teacher_output, inputs))

  def get_eval_loss(self, model, teacher_output, inputs):
    del teacher_output
    return self._standardize_loss_output(self.strategy.get_eval_loss(model, inputs))

  def _log_aux(self, buf, aux) -> None:
    if buf is None or not aux:
      return
    for name, v in aux.items():
      buf.additional_metrics.setdefault(name, ([], np.mean))[0].append(v)

  def _post_process_train_step(self, aux: Any) -> None:
    self._log_aux(self._buffered_train_metrics, aux)

  def _post_process_eval_step(self, aux: Any) -> None:
    self._log_aux(self._buffered_eval_metrics, aux)

  def close(self):
    super().close()
    self.model, self.teacher_model = self.strategy.post_process_models(self.model, self.teacher_model)
