"""Feature-map distillation with average pooling of the teacher's features down to the
student's shape; default feature loss is the mean cosine distance
(tunix/distillation/strategies/feature_pooling.py:30-199)."""
from __future__ import annotations

from typing import Callable, Optional, Sequence, Type, Union

import torch
import torch.nn.functional as F

from .. import feature_extraction as fx
from .base_strategy import BaseStrategy, softmax_cross_entropy


def cosine_distance(a: torch.Tensor, b: torch.Tensor, axis: Union[int, Sequence[int]] = -1,
                    eps: float = 1e-12) -> torch.Tensor:
  axes = (axis,) if isinstance(axis, int) else tuple(axis)
  a, b = a.float(), b.float()
  dot = (a * b).sum(axes)
  na = a.pow(2).sum(axes).clamp_min(eps).sqrt()
  nb = b.pow(2).sum(axes).clamp_min(eps).sqrt()
  return 1.0 - dot / (na * nb)


class FeaturePoolingStrategy(BaseStrategy):
  def __init__(self, student_forward_fn, teacher_forward_fn, labels_fn, feature_layer: Type[torch.nn.Module],
               alpha: float = 0.75, feature_loss_fn: Optional[Callable] = None,
               cosine_distance_axis: Union[int, Sequence[int]] = -1):
    super().__init__(student_forward_fn, teacher_forward_fn, labels_fn)
    if not 0.0 <= alpha <= 1.0:
      raise ValueError(f"Alpha must be a float between 0.0 and 1.0, got {alpha}")
    self.alpha = alpha
    self.feature_loss_fn = feature_loss_fn or (lambda s, t: cosine_distance(s, t, cosine_distance_axis).mean())
    self.feature_layer = feature_layer

  def pre_process_models(self, student_model, teacher_model):
    fx.wrap_model_with_sowed_modules(student_model, [self.feature_layer])
    fx.wrap_model_with_sowed_modules(teacher_model, [self.feature_layer])
    return student_model, teacher_model

  def post_process_models(self, student_model, teacher_model):
    fx.unwrap_sowed_modules(student_model)
    fx.unwrap_sowed_modules(teacher_model)
    return student_model, teacher_model

  def get_teacher_outputs(self, teacher_model, inputs):
    with torch.no_grad():
      self._teacher_forward_fn(teacher_model, **inputs)
    return fx.stack_features(fx.pop_sowed_intermediate_outputs(teacher_model)).detach()

  def get_student_outputs(self, student_model, inputs):
    logits = self._student_forward_fn(student_model, **inputs)
    feats = fx.stack_features(fx.pop_sowed_intermediate_outputs(student_model))
    return {"logits": logits, "features": feats}

  def compute_eval_loss(self, student_output, labels):
    return softmax_cross_entropy(student_output["logits"], labels).mean()

  def compute_loss(self, student_output, teacher_output, labels):
    if not isinstance(student_output, dict) or "logits" not in student_output or "features" not in student_output:
      raise TypeError("student_outputs must be a dict containing 'logits' and 'features'")
    sf = student_output["features"]
    tf = fx.avg_pool_array_to_target_shape(teacher_output, sf.shape)
    feature_loss = self.feature_loss_fn(sf, tf)
    task = softmax_cross_entropy(student_output["logits"], labels).mean()
    return self.alpha * feature_loss + (1.0 - self.alpha) * task
