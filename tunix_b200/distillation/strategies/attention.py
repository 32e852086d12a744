"""Attention-layer variants of the two feature strategies
(tunix/distillation/strategies/attention.py:28-115)."""
from __future__ import annotations

from .feature_pooling import FeaturePoolingStrategy
from .feature_projection import FeatureProjectionStrategy


class AttentionTransferStrategy(FeaturePoolingStrategy):
  def __init__(self, student_forward_fn, teacher_forward_fn, labels_fn, attention_layer, alpha: float = 0.75,
               attention_loss_fn=None):
    super().__init__(student_forward_fn, teacher_forward_fn, labels_fn, feature_layer=attention_layer,
                     alpha=alpha, feature_loss_fn=attention_loss_fn)


class AttentionProjectionStrategy(FeatureProjectionStrategy):
  def __init__(self, student_forward_fn, teacher_forward_fn, labels_fn, attention_layer, dummy_input, rngs=0,
               alpha: float = 0.75, attention_loss_fn=None):
    super().__init__(student_forward_fn, teacher_forward_fn, labels_fn, feature_layer=attention_layer,
                     dummy_input=dummy_input, rngs=rngs, alpha=alpha, feature_loss_fn=attention_loss_fn)
