"""Student wrapper that projects captured features onto the teacher's feature shape.

Role of tunix/distillation/feature_extraction/projection.py:26-140: a learned linear map
contracting every axis of the stacked student features into the stacked teacher feature
shape (a `LinearGeneral` over all axes), trained together with the student.
"""
from __future__ import annotations

import math
from typing import Any, Dict, Sequence, Tuple, Type

import torch

from . import sowed_module


class ModelWithFeatureProjection(torch.nn.Module):
  def __init__(self, model: torch.nn.Module, feature_shape: Sequence[int], feature_target_shape: Sequence[int],
               *, seed: int = 0):
    super().__init__()
    feature_shape = (feature_shape,) if isinstance(feature_shape, int) else tuple(feature_shape)
    feature_target_shape = ((feature_target_shape,) if isinstance(feature_target_shape, int)
                            else tuple(feature_target_shape))
    self.model = model
    self.feature_shape, self.feature_target_shape = feature_shape, feature_target_shape
    n_in, n_out = math.prod(feature_shape), math.prod(feature_target_shape)
    p = next(model.parameters())
    g = torch.Generator().manual_seed(seed)
    w = torch.randn(n_in, n_out, generator=g) / math.sqrt(n_in)     # lecun-normal, as LinearGeneral's default
    self.projection_kernel = torch.nn.Parameter(w.to(device=p.device, dtype=torch.float32))
    self.projection_bias = torch.nn.Parameter(torch.zeros(n_out, device=p.device, dtype=torch.float32))

  def project(self, feats: torch.Tensor) -> torch.Tensor:
    y = feats.reshape(-1).float() @ self.projection_kernel + self.projection_bias
    return y.reshape(self.feature_target_shape)

  def forward(self, *args, **kwargs):
    output = self.model(*args, **kwargs)
    feats = sowed_module.stack_features(sowed_module.pop_sowed_intermediate_outputs(self.model))
    return output, self.project(feats)

  def __getattr__(self, name):          # config, init_cache, ... of the wrapped model stay reachable
    try:
      return super().__getattr__(name)
    except AttributeError:
      return getattr(super().__getattr__("model"), name)


def setup_models_with_feature_projection(student_model, teacher_model, student_layer_to_capture: Type,
                                         teacher_layer_to_capture: Type, dummy_student_input: Dict[str, Any],
                                         dummy_teacher_input: Dict[str, Any], *, seed: int = 0
                                         ) -> Tuple[ModelWithFeatureProjection, torch.nn.Module]:
  sowed_module.wrap_model_with_sowed_modules(student_model, [student_layer_to_capture])
  sowed_module.wrap_model_with_sowed_modules(teacher_model, [teacher_layer_to_capture])
  with torch.no_grad():
    student_model(**dummy_student_input)
    teacher_model(**dummy_teacher_input)
  sf = sowed_module.stack_features(sowed_module.pop_sowed_intermediate_outputs(student_model))
  tf = sowed_module.stack_features(sowed_module.pop_sowed_intermediate_outputs(teacher_model))
  return ModelWithFeatureProjection(student_model, sf.shape, tf.shape, seed=seed), teacher_model


def remove_feature_projection_from_models(student_model, teacher_model):
  if isinstance(student_model, ModelWithFeatureProjection):
    student_model = student_model.model
  sowed_module.unwrap_sowed_modules(student_model)
  sowed_module.unwrap_sowed_modules(teacher_model)
  return student_model, teacher_model
