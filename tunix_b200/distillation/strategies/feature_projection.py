"""Feature-map distillation through a learned projection of the student's features onto the
teacher's feature shape; default feature loss is MSE
(tunix/distillation/strategies/feature_projection.py:30-198)."""
from __future__ import annotations

from typing import Any, Callable, Dict, Optional, Type

import torch

from .. import feature_extraction as fx
from .base_strategy import BaseStrategy, softmax_cross_entropy


class FeatureProjectionStrategy(BaseStrategy):
  def __init__(self, student_forward_fn, teacher_forward_fn, labels_fn, feature_layer: Type[torch.nn.Module],
               dummy_input: Dict[str, Any], rngs: Any = 0, alpha: float = 0.75,
               feature_loss_fn: Optional[Callable] = None):
    super().__init__(student_forward_fn, teacher_forward_fn, labels_fn)
    if not 0.0 <= alpha <= 1.0:
      raise ValueError(f"Alpha must be a float between 0.0 and 1.0, got {alpha}")
    self.alpha = alpha
    self.feature_loss_fn = feature_loss_fn or (lambda s, t: (s.float() - t.float()).pow(2).mean())
    self.feature_layer, self.dummy_input = feature_layer, dummy_input
    self.seed = int(rngs) if isinstance(rngs, int) else 0

  def pre_process_models(self, student_model, teacher_model):
    return fx.setup_models_with_feature_projection(student_model, teacher_model, self.feature_layer,
                                                   self.feature_layer, self.dummy_input, self.dummy_input,
                                                   seed=self.seed)

  def post_process_models(self, student_model, teacher_model):
    return fx.remove_feature_projection_from_models(student_model, teacher_model)

  def get_teacher_outputs(self, teacher_model, inputs):
    with torch.no_grad():
      self._teacher_forward_fn(teacher_model, **inputs)
    return fx.stack_features(fx.pop_sowed_intermediate_outputs(teacher_model)).detach()

  def get_student_outputs(self, student_model, inputs):
    logits, feats = self._student_forward_fn(student_model, **inputs)
    return {"logits": logits, "features": feats}

  def compute_eval_loss(self, student_output, labels):
    return softmax_cross_entropy(student_output["logits"], labels).mean()

  def compute_loss(self, student_output, teacher_output, labels):
    if not isinstance(student_output, dict) or "logits" not in student_output or "features" not in student_output:
      raise TypeError("student_outputs must be a dict containing 'logits' and 'features'")
    feature_loss = self.feature_loss_fn(student_output["features"], teacher_output)
    task = softmax_cross_entropy(student_output["logits"], labels).mean()
    return self.alpha * feature_loss + (1.0 - self.alpha) * task
