"""More trainer semantics: the gradient accumulator by itself, data-driven update cadence, denominators that are
global over micro-batches, metric reduction rules, trainer reuse, resumption that skips consumed batches, and
max_steps."""
import numpy as np
import pytest
import torch

from tunix_b200 import optim
from tunix_b200.sft import peft_trainer as pt
from tunix_b200.sft.peft_trainer import GradientAccumulator, MetricsBuffer, PeftTrainer, TrainingInput
from tunix_b200.sft.utils import LossOutput, WeightedMetric
from tests.test_sft_trainer import batches, cfg, tiny


# ---- the accumulator by itself ----------------------------------------------------------------------
def _params():
  return {"w": torch.nn.Parameter(torch.zeros(3)), "b": torch.nn.Parameter(torch.zeros(()))}


def test_accumulator_sums_gradients_and_denominators_and_divides_once():
  ps = _params()
  acc = GradientAccumulator(ps)
  for g, d in ((torch.tensor([1.0, 2.0, 3.0]), 2.0), (torch.tensor([3.0, 2.0, 1.0]), torch.tensor(6.0))):
    ps["w"].grad, ps["b"].grad = g.clone(), torch.tensor(1.0)
    acc.collect(d)
    assert ps["w"].grad is None                                  # folded in and cleared
  assert acc.acc["w"].tolist() == [4.0, 4.0, 4.0] and float(acc.acc["b"]) == 2.0 and float(acc.denom) == 8.0
  assert float(acc.get_scale()) == pytest.approx(1 / 8)
  assert acc.acc["w"].dtype == torch.float32
  acc.reset()
  assert float(acc.denom) == 0.0 and not acc.acc["w"].any() and float(acc.get_scale()) == 0.0     # zero-safe


def test_accumulator_keeps_fp32_for_low_precision_parameters_and_skips_missing_grads():
  ps = {"h": torch.nn.Parameter(torch.zeros(4, dtype=torch.bfloat16)), "unused": torch.nn.Parameter(torch.zeros(2))}
  acc = GradientAccumulator(ps)
  for _ in range(300):
    ps["h"].grad = torch.full((4,), 0.001, dtype=torch.bfloat16)
    acc.collect(1.0)
  assert acc.acc["h"].dtype == torch.float32
  assert float(acc.acc["h"][0]) == pytest.approx(300 * float(torch.tensor(0.001, dtype=torch.bfloat16)), rel=1e-5)
  assert not acc.acc["unused"].any()


def test_accumulator_leaves_store_managed_parameters_alone():
  p = torch.nn.Parameter(torch.zeros(2))
  p.grad_managed = True
  acc = GradientAccumulator({"managed": p, "plain": torch.nn.Parameter(torch.zeros(2))})
  assert list(acc.acc) == ["plain"]
  p.grad = torch.ones(2)
  acc.collect(1.0)
  assert p.grad is not None                                      # not folded: its store does that


# ---- update cadence -----------------------------------------------------------------------------------
def test_zero_denominator_step_changes_nothing():
  model = tiny()
  before = {n: p.detach().clone() for n, p in model.named_parameters()}
  tr = PeftTrainer(model, optim.adam(1e-2), cfg())          # no weight decay: only gradients could move a weight
  data = [TrainingInput(b.input_tokens, torch.zeros_like(b.input_mask)) for b in batches(2)]
  tr.train(data)
  assert tr.train_steps == 2
  for n, p in model.named_parameters():
    assert torch.equal(p, before[n]), n
  assert all(np.isfinite(v) for v in tr.metrics_logger.get_metric_history("", "loss", "train"))


def test_data_driven_update_flag_overrides_the_accumulation_count():
  """Batches that carry `is_update_step` (the sequence packer's) decide when the optimizer steps: 1 + 3 + 2
  micro-batches give three updates, whatever gradient_accumulation_steps says."""
  flags = [True, False, False, True, False, True]
  data = [{"input_tokens": b.input_tokens, "input_mask": b.input_mask, "is_update_step": torch.tensor([f])}
          for b, f in zip(batches(6), flags)]
  seen = []

  def loss_fn(model, input_tokens, input_mask, **kw):
    seen.append(1)
    logits = model(input_tokens)[0]
    ce = torch.nn.functional.cross_entropy(logits[:, :-1].reshape(-1, logits.shape[-1]).float(),
                                           input_tokens[:, 1:].reshape(-1), reduction="sum")
    return LossOutput(WeightedMetric(ce, input_mask[:, 1:].sum()), {})
  tr = PeftTrainer(tiny(), optim.adamw(1e-3), cfg(gradient_accumulation_steps=4))
  tr.with_loss_fn(loss_fn).with_gen_model_input_fn(lambda x: {k: v for k, v in x.items() if k != "is_update_step"})
  tr.train(data)
  assert tr.train_steps == 3 and tr.iter_steps == 6 and len(seen) == 6
  assert len(tr.metrics_logger.get_metric_history("", "loss", "train")) == 3


def test_reported_loss_uses_the_global_denominator_of_the_step():
  """Two micro-batches with 4 and 12 loss tokens: the step's loss is sum(ce) / 16, not the mean of two means; the
  update equals the one of the concatenated batch."""
  b = batches(1, B=4, L=9, seed=5)[0]
  small = TrainingInput(b.input_tokens[:2], torch.cat([torch.ones(2, 3), torch.zeros(2, 6)], 1))
  large = TrainingInput(b.input_tokens[2:], torch.cat([torch.ones(2, 7), torch.zeros(2, 2)], 1))
  whole = TrainingInput(b.input_tokens, torch.cat([small.input_mask, large.input_mask]))
  runs = []
  for data, ga in (([small, large], 2), ([whole], 1)):
    model = tiny(seed=3)
    tr = PeftTrainer(model, optim.adamw(1e-2), cfg(gradient_accumulation_steps=ga))
    tr.train(data)
    runs.append((tr.metrics_logger.get_metric_history("", "loss", "train")[0],
                 {n: p.detach().clone() for n, p in model.named_parameters()}))
  assert runs[0][0] == pytest.approx(runs[1][0], rel=1e-5)
  for n in runs[0][1]:
    torch.testing.assert_close(runs[0][1][n], runs[1][1][n], rtol=1e-4, atol=1e-6)


def test_max_steps_stops_the_loop_unless_the_trainer_is_driven_from_outside():
  tr = PeftTrainer(tiny(), optim.adamw(1e-3), cfg(max_steps=3))
  tr.train(batches(10))
  assert tr.train_steps == 3 and tr.iter_steps == 3
  tr.train(batches(10, seed=1))                     # the budget is spent: a second call trains nothing
  assert tr.train_steps == 3
  outer = PeftTrainer(tiny(), optim.adamw(1e-3), cfg(max_steps=3))
  outer.is_managed_externally = True                # an RL learner owns the stopping rule and the trainer's life
  outer.train(batches(5))
  outer.train(batches(2, seed=1))
  assert outer.train_steps == 7
  outer.close()                                     # the last step's metrics are read back lazily: close flushes them
  assert len(outer.metrics_logger.get_metric_history("", "loss", "train")) == 7


def test_resume_skips_the_batches_already_consumed(tmp_path):
  """A second trainer over the same data directory and dataset continues where the first stopped: it must
  not train on the first batches again."""
  data = batches(6, seed=2)
  a = PeftTrainer(tiny(), optim.adamw(1e-2), cfg(max_steps=3, checkpoint_root_directory=str(tmp_path)))
  a.train(data)
  consumed = []
  b = PeftTrainer(tiny(), optim.adamw(1e-2), cfg(max_steps=6, checkpoint_root_directory=str(tmp_path)))
  assert b.train_steps == 3
  b.with_gen_model_input_fn(lambda x: (consumed.append(x.input_tokens), {"input_tokens": x.input_tokens,
                                                                        "input_mask": x.input_mask})[1])
  b.train(data)
  assert b.train_steps == 6 and len(consumed) == 3
  assert all(torch.equal(c.cpu(), d.input_tokens) for c, d in zip(consumed, data[3:]))
  straight = PeftTrainer(tiny(), optim.adamw(1e-2), cfg(max_steps=6))
  straight.train(data)
  for (n, p), (_, q) in zip(b.model.named_parameters(), straight.model.named_parameters()):
    torch.testing.assert_close(p, q, rtol=1e-4, atol=1e-6, msg=n)


# ---- metric reduction -----------------------------------------------------------------------------------
def test_weighted_metrics_reduce_globally_scalars_by_mean_and_kinds_do_not_mix():
  ms = [WeightedMetric(torch.tensor(2.0), torch.tensor(1.0)), WeightedMetric(torch.tensor(6.0), torch.tensor(3.0))]
  assert pt._weighted_metric_mean(ms) == pytest.approx(2.0)             # 8 / 4, not (2 + 2) / 2 by accident
  ms2 = [WeightedMetric(4.0, 1.0), WeightedMetric(6.0, 9.0)]
  assert pt._weighted_metric_mean(ms2) == pytest.approx(1.0)            # 10 / 10; the mean of means would be 2.33
  assert pt._metric_reducer(ms[0]) is pt._weighted_metric_mean and pt._metric_reducer(1.0) is np.mean
  assert MetricsBuffer(step=0, losses=ms2).loss == pytest.approx(1.0)
  assert MetricsBuffer(step=0, losses=[1.0, torch.tensor(3.0)]).loss == 2.0
  # bounds on the denominator survive the reduction
  bounded = [WeightedMetric(1.0, 0.0, min_denom=2.0), WeightedMetric(1.0, 0.0, min_denom=2.0)]
  assert pt._weighted_metric_mean(bounded) == pytest.approx(1.0)        # 2 / max(0, 2)
  assert float(WeightedMetric(5.0, 0.0).compute()) == 0.0


def test_aux_metrics_are_logged_with_their_own_reducers():
  def loss_fn(model, input_tokens, input_mask, **kw):
    logits = model(input_tokens)[0]
    ce = torch.nn.functional.cross_entropy(logits[:, :-1].reshape(-1, logits.shape[-1]).float(),
                                           input_tokens[:, 1:].reshape(-1), reduction="none")
    m = input_mask[:, 1:].reshape(-1)
    tokens = m.sum()
    return LossOutput(WeightedMetric((ce * m).sum(), tokens),
                      {"tokens_per_micro": tokens.float(), "weighted_one": WeightedMetric(tokens.float(), tokens)})
  tr = PeftTrainer(tiny(), optim.adamw(1e-3), cfg(gradient_accumulation_steps=2))
  tr.with_loss_fn(loss_fn)
  data = batches(2, ragged=True, seed=4)
  tr.train(data)
  lg = tr.metrics_logger
  per_micro = [float(b.input_mask[:, 1:].sum()) for b in data]
  assert lg.get_metric_history("", "tokens_per_micro", "train")[0] == pytest.approx(np.mean(per_micro))
  assert lg.get_metric_history("", "weighted_one", "train")[0] == pytest.approx(1.0)
  assert lg.metric_exists("", "grad_norm", "train")
