"""Distillation pieces by hand: the cross entropy helper, the logit strategy (temperature, alpha, top-k, metrics),
cosine distance and the pooling strategy's mix, pooling windows in both padding modes, and feature capture
(wrap / pop / unwrap) on plain modules."""
import math

import pytest
import torch
import torch.nn.functional as F

from tunix_b200.distillation import feature_extraction as fx, strategies
from tunix_b200.distillation.feature_extraction import pooling
from tunix_b200.distillation.strategies import base_strategy, feature_pooling


def make_logit(**kw):
  return strategies.LogitStrategy(lambda m, **i: None, lambda m, **i: None, lambda **i: None, **kw)


def test_cross_entropy_takes_ids_one_hot_and_soft_labels():
  logits = torch.tensor([[[2.0, 0.0, -1.0], [0.0, 0.0, 0.0]]])
  ids = torch.tensor([[0, 2]])
  by_id = base_strategy.softmax_cross_entropy(logits, ids)
  assert by_id.shape == (1, 2) and float(by_id[0, 1]) == pytest.approx(math.log(3))
  torch.testing.assert_close(base_strategy.softmax_cross_entropy(logits, F.one_hot(ids, 3).float()), by_id)
  soft = torch.tensor([[[0.5, 0.5, 0.0], [1 / 3, 1 / 3, 1 / 3]]])
  lp = F.log_softmax(logits, -1)
  assert float(base_strategy.softmax_cross_entropy(logits, soft)[0, 0]) == pytest.approx(float(-(0.5 * lp[0, 0, 0] + 0.5 * lp[0, 0, 1])))


def test_logit_strategy_by_hand():
  s = torch.tensor([[[1.0, 0.0, -1.0, 0.5]]])
  t = torch.tensor([[[2.0, 1.0, 0.0, -2.0]]])
  labels = torch.tensor([[1]])
  tau, alpha = 2.0, 0.3
  loss, aux = make_logit(temperature=tau, alpha=alpha).compute_loss(s, t, labels)
  ps, pt = F.softmax(s / tau, -1), F.softmax(t / tau, -1)
  kl = float((pt * (pt.log() - ps.log())).sum())
  hard = float(-F.log_softmax(s, -1)[0, 0, 1])
  assert float(aux["distill/kl_div"]) == pytest.approx(kl, rel=1e-5)
  assert float(aux["distill/soft_loss"]) == pytest.approx(kl * tau ** 2, rel=1e-5)      # gradients keep their scale
  assert float(aux["distill/hard_loss"]) == pytest.approx(hard, rel=1e-5)
  assert float(aux["distill/teacher_loss"]) == pytest.approx(float(-F.log_softmax(t, -1)[0, 0, 1]), rel=1e-5)
  assert float(loss) == pytest.approx(alpha * kl * tau ** 2 + (1 - alpha) * hard, rel=1e-5)
  # identical logits: nothing to distil; alpha picks the mixture's ends
  same, aux_same = make_logit(alpha=1.0).compute_loss(t, t, labels)
  assert float(same) == pytest.approx(0.0, abs=1e-6)
  only_task, _ = make_logit(alpha=0.0).compute_loss(s, t, labels)
  assert float(only_task) == pytest.approx(hard, rel=1e-5)
  ev = make_logit().compute_eval_loss(s, labels)
  assert float(ev[0]) == pytest.approx(hard, rel=1e-5) and ev[1] == {}


def test_top_k_distillation_renormalises_over_the_teachers_best_logits():
  s = torch.tensor([[[1.0, 0.0, -1.0, 0.5]]])
  t = torch.tensor([[[2.0, 1.0, 0.0, -2.0]]])
  _, aux = make_logit(temperature=1.0, distill_top_k=2).compute_loss(s, t, torch.tensor([[0]]))
  pt = F.softmax(torch.tensor([2.0, 1.0]), -1)                  # teacher's top two: classes 0 and 1
  ps = F.softmax(torch.tensor([1.0, 0.0]), -1)                  # the student's logits at those classes
  assert float(aux["distill/kl_div"]) == pytest.approx(float((pt * (pt.log() - ps.log())).sum()), rel=1e-5)
  full = make_logit(temperature=1.0).compute_loss(s, t, torch.tensor([[0]]))[1]["distill/kl_div"]
  assert float(full) != pytest.approx(float(aux["distill/kl_div"]))
  with pytest.raises(ValueError, match="Temperature must be a positive"):
    make_logit(temperature=0.0)
  with pytest.raises(ValueError, match="Alpha must be"):
    make_logit(alpha=1.5)


def test_gradients_reach_the_student_only():
  s = torch.randn(2, 3, 5, requires_grad=True)
  t = torch.randn(2, 3, 5, requires_grad=True)
  loss, _ = make_logit().compute_loss(s, t.detach(), torch.randint(0, 5, (2, 3)))
  loss.backward()
  assert s.grad is not None and s.grad.abs().sum() > 0 and t.grad is None


def test_cosine_distance_axes_and_zero_vectors():
  a = torch.tensor([[1.0, 0.0], [1.0, 1.0], [0.0, 0.0]])
  b = torch.tensor([[0.0, 2.0], [2.0, 2.0], [1.0, 0.0]])
  d = feature_pooling.cosine_distance(a, b)
  assert d.tolist() == pytest.approx([1.0, 0.0, 1.0], abs=1e-6)          # orthogonal, parallel, undefined -> 1
  whole = feature_pooling.cosine_distance(a, b, axis=(0, 1))
  assert float(whole) == pytest.approx(1 - 4 / (math.sqrt(3) * math.sqrt(13)), rel=1e-6)


def test_pooling_strategy_mixes_feature_and_task_loss():
  strat = strategies.FeaturePoolingStrategy(lambda m, **i: None, lambda m, **i: None, lambda **i: None,
                                            feature_layer=torch.nn.Linear, alpha=0.25)
  student = {"logits": torch.tensor([[[2.0, 0.0]]]), "features": torch.tensor([[[1.0, 0.0]]])}
  teacher = torch.tensor([[[0.0, 1.0, 0.0, 3.0]]])                        # pooled in pairs to [0.5, 1.5]
  labels = torch.tensor([[0]])
  got = strat.compute_loss(student, teacher, labels)
  feature = 1 - 0.5 / math.sqrt(0.25 + 2.25)
  task = float(-F.log_softmax(student["logits"], -1)[0, 0, 0])
  assert float(got) == pytest.approx(0.25 * feature + 0.75 * task, rel=1e-5)
  assert float(strat.compute_eval_loss(student, labels)) == pytest.approx(task, rel=1e-5)
  with pytest.raises(TypeError, match="'logits' and 'features'"):
    strat.compute_loss(student["logits"], teacher, labels)
  mse = strategies.FeaturePoolingStrategy(lambda m, **i: None, lambda m, **i: None, lambda **i: None,
                                          feature_layer=torch.nn.Linear, alpha=1.0,
                                          feature_loss_fn=lambda s, t: (s - t).pow(2).mean())
  assert float(mse.compute_loss(student, teacher, labels)) == pytest.approx((0.25 + 2.25) / 2, rel=1e-6)


def test_pooling_windows_in_both_padding_modes():
  x = torch.arange(1.0, 8.0)[None]                                         # [1, 7]
  valid = pooling.avg_pool_array_to_target_shape(x, (1, 3))
  # VALID: stride 7 // 3 = 2, window 7 - 2 * 2 = 3 -> [1,2,3], [3,4,5], [5,6,7]
  assert valid.tolist() == [[2.0, 4.0, 6.0]]
  same = pooling.avg_pool_array_to_target_shape(x, (1, 3), pooling.PaddingMode.SAME)
  # SAME: window = stride = 3, two padded slots split 1 / 1 -> [_,1,2], [3,4,5], [6,7,_]; real elements only
  assert same.tolist() == [[1.5, 4.0, 6.5]]
  counted = pooling.avg_pool_array_to_target_shape(x, (1, 3), pooling.PaddingMode.SAME, True)
  assert counted.tolist() == [[1.0, 4.0, pytest.approx(13 / 3)]]
  assert pooling.avg_pool_array_to_target_shape(x, (1, 7)) is x
  grid = torch.arange(16.0).view(1, 4, 4)
  assert pooling.avg_pool_array_to_target_shape(grid, (1, 2, 2)).tolist() == [[[2.5, 4.5], [10.5, 12.5]]]
  with pytest.raises(ValueError, match="rank"):
    pooling.avg_pool_array_to_target_shape(x, (3,))
  with pytest.raises(ValueError, match="Must be 1 <= target_dim"):
    pooling.avg_pool_array_to_target_shape(x, (1, 9))


def test_feature_capture_wraps_pops_and_unwraps():
  class Net(torch.nn.Module):
    def __init__(self):
      super().__init__()
      self.a, self.b, self.act = torch.nn.Linear(3, 4), torch.nn.Linear(4, 4), torch.nn.Tanh()
    def forward(self, x):
      return self.b(self.act(self.a(x)))
  net = Net()
  x = torch.randn(2, 3)
  plain = net(x)
  fx.wrap_model_with_sowed_modules(net, [torch.nn.Linear])
  wrapped = net(x)
  torch.testing.assert_close(wrapped, plain)                               # capturing changes no values
  feats = fx.pop_sowed_intermediate_outputs(net)
  assert len(feats) == 2 and all(v.shape == (2, 4) for v in feats.values())
  assert fx.stack_features(feats).shape[0] == 2
  assert fx.pop_sowed_intermediate_outputs(net) == {}                      # popping empties the store
  fx.unwrap_sowed_modules(net)
  fx.unwrap_sowed_modules(net)                                             # idempotent
  torch.testing.assert_close(net(x), plain)
  with pytest.raises(ValueError, match="no capture hooks"):
    fx.pop_sowed_intermediate_outputs(net)                                 # nothing is captured any more
  with pytest.raises(ValueError, match="no sub-module of type"):
    fx.wrap_model_with_sowed_modules(net, [torch.nn.Conv2d])
