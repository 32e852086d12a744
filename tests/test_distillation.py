"""Distillation trainer and strategies on CPU."""
import numpy as np
import pytest
import torch
import torch.nn.functional as F

from tunix_b200 import optim
from tunix_b200.common.configs import TrainingConfig
from tunix_b200.distillation import DistillationTrainer, TrainingInput, feature_extraction as fx, strategies
from tunix_b200.models.transformer import ModelConfig, Transformer
from tunix_b200.sft import utils as sft_utils


def model(layers, embed, seed):
  cfg = ModelConfig(num_layers=layers, vocab_size=48, embed_dim=embed, hidden_dim=2 * embed, num_heads=4,
                    head_dim=embed // 4, num_kv_heads=2)
  return Transformer(cfg).init_weights(seed=seed, scale=0.2)


def fwd(m, input_tokens, input_mask):
  pos = sft_utils.build_positions_from_mask(input_mask)
  attn = sft_utils.make_causal_attn_mask(input_mask)
  out = m(input_tokens, pos, None, attn)
  if isinstance(out[0], tuple):     # projection wrapper: ((logits, cache), features)
    return out[0][0], out[1]
  return out[0]


def labels(input_tokens, input_mask):
  return F.one_hot(torch.roll(input_tokens, -1, 1), 48).float()


def data(n):
  g = torch.Generator().manual_seed(0)
  return [TrainingInput(torch.randint(1, 48, (2, 8), generator=g), torch.ones(2, 8, dtype=torch.long))
          for _ in range(n)]


def cfg(steps):
  return TrainingConfig(eval_every_n_steps=100, max_steps=steps, pbar_description=None)


def test_avg_pool_matches_torch_pooling():
  x = torch.arange(2 * 12 * 10, dtype=torch.float32).reshape(2, 12, 10)
  y = fx.avg_pool_array_to_target_shape(x, (2, 4, 5))
  want = F.avg_pool2d(x[None], (3, 2), (3, 2))[0]
  torch.testing.assert_close(y, want)
  y = fx.avg_pool_array_to_target_shape(x, (1, 5, 10))       # VALID: stride 2, window 4 on axis 1
  want = torch.stack([x[:, 2 * i:2 * i + 4].mean(1) for i in range(5)], 1).mean(0, keepdim=True)
  torch.testing.assert_close(y, want)
  y = fx.avg_pool_array_to_target_shape(x, (2, 5, 10), fx.PaddingMode.SAME)   # stride 3, pad 3 -> lo 1
  assert y.shape == (2, 5, 10)
  torch.testing.assert_close(y[:, 0], x[:, 0:2].mean(1))
  with pytest.raises(ValueError):
    fx.avg_pool_array_to_target_shape(x, (2, 13, 10))


def test_logit_strategy_values_and_training():
  s = strategies.LogitStrategy(fwd, fwd, labels, temperature=2.0, alpha=0.5)
  sl, tl = torch.randn(2, 3, 48), torch.randn(2, 3, 48)
  lab = F.one_hot(torch.randint(0, 48, (2, 3)), 48).float()
  loss, m = s.compute_loss(sl, tl, lab)
  kl = F.kl_div(F.log_softmax(sl / 2, -1), F.softmax(tl / 2, -1), reduction="none").sum(-1)
  ce = F.cross_entropy(sl.reshape(-1, 48), lab.argmax(-1).reshape(-1))
  torch.testing.assert_close(loss, 0.5 * 4 * kl.mean() + 0.5 * ce)
  torch.testing.assert_close(m["distill/kl_div"], kl.mean())
  sk = strategies.LogitStrategy(fwd, fwd, labels, distill_top_k=5)
  assert sk.compute_loss(sl, tl, lab)[0].isfinite()
  with pytest.raises(ValueError):
    strategies.LogitStrategy(fwd, fwd, labels, temperature=0)
  student, teacher = model(1, 16, 0), model(2, 32, 1)
  tr = DistillationTrainer(student, teacher, s, optim.adamw(1e-2), cfg(5))
  with pytest.raises(NotImplementedError):
    tr.with_loss_fn(lambda *a: 0)
  tr.train(data(5), data(1))
  soft = tr.metrics_logger.get_metric_history("", "distill/soft_loss", "train")
  assert len(soft) == 5 and soft[-1] < soft[0]
  assert tr.metrics_logger.metric_exists("", "loss", "eval")


@pytest.mark.parametrize("kind", ["pooling", "projection", "attn_transfer", "attn_projection"])
def test_feature_strategies_train_and_unwrap(kind):
  from tunix_b200.models.transformer import Attention, DecoderLayer
  student, teacher = model(2, 16, 0), model(2, 32, 1)
  ones = torch.ones(2, 8, dtype=torch.long)
  dummy = {"input_tokens": ones, "positions": sft_utils.build_positions_from_mask(ones), "cache": None,
           "attention_mask": sft_utils.make_causal_attn_mask(ones)}
  if kind == "pooling":
    s = strategies.FeaturePoolingStrategy(fwd, fwd, labels, DecoderLayer)
  elif kind == "projection":
    s = strategies.FeatureProjectionStrategy(fwd, fwd, labels, DecoderLayer, dummy, 0)
  elif kind == "attn_transfer":
    s = strategies.AttentionTransferStrategy(fwd, fwd, labels, Attention)
  else:
    s = strategies.AttentionProjectionStrategy(fwd, fwd, labels, Attention, dummy, 0)
  n_params = sum(1 for _ in student.parameters())
  tr = DistillationTrainer(student, teacher, s, optim.adamw(5e-3), cfg(4))
  tr.train(data(4), data(1))
  l = tr.metrics_logger.get_metric_history("", "loss", "train")
  assert len(l) == 4 and l[-1] < l[0]
  assert tr.model is student and sum(1 for _ in tr.model.parameters()) == n_params
  assert getattr(student, "_sowed_state", None) is None and getattr(teacher, "_sowed_state", None) is None
