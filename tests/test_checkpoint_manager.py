"""`CheckpointManager` and its options on one process: nothing without a root, policies (interval, time, force,
preservation), synchronous and asynchronous writes, atomic commit, restore of model / LoRA subset / optimizer state
/ custom metadata, and the error for restoring everything from an adapters-only checkpoint."""
import os
import time
import types

import pytest
import torch

from tunix_b200 import optim
from tunix_b200.models import lora as lora_lib
from tunix_b200.sft import checkpoint_manager as cm, checkpoint_options as co
from tunix_b200.sft.peft_trainer import ModelOptimizer
from tests.test_sft_trainer import tiny


def options(**kw):
  kw.setdefault("save_decision_policy", co.FixedIntervalPolicy(1))
  kw.setdefault("enable_async_checkpointing", False)
  return co.TunixCheckpointingOptions(**kw)


def perturbed(seed):
  model = tiny()
  g = torch.Generator().manual_seed(seed)
  with torch.no_grad():
    for p in model.parameters():
      p.add_(0.1 * torch.randn(p.shape, generator=g))
  return model


def same(a, b):
  return all(torch.equal(p, q) for (_, p), (_, q) in zip(a.named_parameters(), b.named_parameters()))


def test_without_a_root_directory_nothing_happens():
  mgr = cm.CheckpointManager(None)
  assert mgr.latest_step() is None and mgr.all_steps() == []
  assert mgr.save(1, tiny()) is False and mgr.maybe_restore(tiny()) == (0, {})
  mgr.close()
  assert cm.CheckpointManager("").latest_step() is None


def test_defaults_are_filled_in_and_legacy_fields_understood():
  d = co.resolve_checkpointing_defaults(None)
  assert isinstance(d.save_decision_policy, co.ContinuousCheckpointingPolicy) and d.preservation_policy == co.LatestN(3)
  assert d.enable_async_checkpointing and d.async_options.timeout_secs == 1200
  partial = co.resolve_checkpointing_defaults(co.TunixCheckpointingOptions(enable_async_checkpointing=False))
  assert partial.enable_async_checkpointing is False and partial.preservation_policy == co.LatestN(3)
  legacy = co.resolve_checkpointing_defaults(types.SimpleNamespace(save_interval_steps=5, max_to_keep=2))
  assert legacy.save_decision_policy == co.FixedIntervalPolicy(5) and legacy.preservation_policy == co.LatestN(2)
  built = co.checkpointing_options_from_dict({"save_interval_steps": 4, "max_to_keep": 1, "timeout_secs": 30})
  assert built.save_decision_policy.interval == 4 and built.async_options.timeout_secs == 30
  assert co.checkpointing_options_from_dict({}) is None
  with pytest.raises(ValueError, match="Unsupported checkpointing options"):
    co.checkpointing_options_from_dict({"save_every": 3})


def test_policies_by_themselves():
  fixed = co.FixedIntervalPolicy(3)
  assert [s for s in range(1, 10) if fixed.should_save(s, None, None)] == [3, 6, 9]
  timed = co.ContinuousCheckpointingPolicy(minimum_interval_secs=100)
  assert timed.should_save(1, None, None) and not timed.should_save(2, 1, time.time() - 5)
  assert timed.should_save(3, 1, time.time() - 101) and co.ContinuousCheckpointingPolicy().should_save(2, 1, time.time())
  assert co.LatestN(2).to_delete([5, 1, 3, 9]) == [1, 3] and co.LatestN(None).to_delete([1, 2, 3]) == []
  assert co.LatestN(5).to_delete([1, 2]) == []


@pytest.mark.parametrize("use_async", [False, True])
def test_saves_follow_the_policy_force_overrides_it_and_old_steps_are_pruned(tmp_path, use_async):
  mgr = cm.CheckpointManager(str(tmp_path), options(save_decision_policy=co.FixedIntervalPolicy(2),
                                                    preservation_policy=co.LatestN(2),
                                                    enable_async_checkpointing=use_async))
  model = tiny()
  saved = [s for s in range(1, 8) if mgr.save(s, model)]
  assert saved == [2, 4, 6]
  assert mgr.save(7, model, force=True) and not mgr.save(7, model, force=True)      # the same step is not rewritten
  mgr.wait_until_finished()
  assert mgr.all_steps() == [6, 7] and mgr.latest_step() == 7                        # LatestN(2) pruned 2 and 4
  assert not [d for d in os.listdir(tmp_path) if ".tmp-" in d]                       # commits are renames
  mgr.close()
  assert cm.CheckpointManager(str(tmp_path)).latest_step() == 7                      # visible to a new manager


def test_model_round_trip_specific_step_and_custom_metadata(tmp_path):
  mgr = cm.CheckpointManager(str(tmp_path), options(preservation_policy=co.LatestN(5)))
  first, second = perturbed(1), perturbed(2)
  mgr.save(1, first, custom_metadata={"global_step": 10, "role": "actor"})
  mgr.save(2, second, custom_metadata={"global_step": 20})
  into = tiny()
  assert mgr.maybe_restore(into) == (2, {"global_step": 20}) and same(into, second)
  assert mgr.maybe_restore(into, step=1) == (1, {"global_step": 10, "role": "actor"}) and same(into, first)
  with pytest.raises(Exception):
    mgr.maybe_restore(into, step=3)
  mgr.close()


def test_optimizer_state_round_trip_and_restore_without_an_optimizer(tmp_path):
  model = perturbed(3)
  opt = ModelOptimizer(model, optim.adamw(1e-2), lora_only=False)
  loss = model(torch.randint(0, 128, (2, 8), generator=torch.Generator().manual_seed(0)))[0].float().pow(2).mean()
  loss.backward()
  opt.update({n: p.grad for n, p in opt.named_params.items()})
  assert opt.step == 1
  mgr = cm.CheckpointManager(str(tmp_path), options())
  mgr.save(1, model, opt)
  fresh_model = tiny()
  fresh = ModelOptimizer(fresh_model, optim.adamw(1e-2), lora_only=False)
  assert mgr.maybe_restore(fresh_model, fresh)[0] == 1 and same(fresh_model, model) and fresh.step == 1
  for key in ("mu", "nu"):
    for n in opt.opt_state[key]:
      torch.testing.assert_close(fresh.opt_state[key][n], opt.opt_state[key][n])
  only_model = tiny()
  assert mgr.maybe_restore(only_model)[0] == 1 and same(only_model, model)          # the optimizer part is optional
  mgr.close()


def test_lora_only_checkpoints(tmp_path):
  torch.manual_seed(0)
  model = tiny()
  lora_lib.apply_lora_to_model(model, rank=2, alpha=4.0)
  with torch.no_grad():
    for n, p in model.named_parameters():
      if getattr(p, "is_lora", False):
        p.add_(0.3)
  mgr = cm.CheckpointManager(str(tmp_path), options())
  mgr.save(1, model, save_only_lora_params=True)
  torch.manual_seed(1)
  other = tiny(seed=9)                                   # another backbone: it must stay untouched
  lora_lib.apply_lora_to_model(other, rank=2, alpha=4.0)
  backbone = {n: p.detach().clone() for n, p in other.named_parameters() if not getattr(p, "is_lora", False)}
  assert mgr.maybe_restore(other, restore_only_lora_params=True)[0] == 1
  for (n, p), (_, q) in zip(other.named_parameters(), model.named_parameters()):
    if getattr(p, "is_lora", False):
      assert torch.equal(p, q), n
    else:
      assert torch.equal(p, backbone[n]), n
  with pytest.raises(ValueError, match="restore_only_lora_params=True"):
    mgr.maybe_restore(other)                             # the full model is not in an adapters-only checkpoint
  mgr.close()


def test_async_write_finishes_before_the_next_decision_and_on_close(tmp_path):
  mgr = cm.CheckpointManager(str(tmp_path), options(enable_async_checkpointing=True,
                                                    save_decision_policy=co.ContinuousCheckpointingPolicy()))
  slow_write = mgr._write

  def delayed(*args, **kw):
    time.sleep(0.3)
    return slow_write(*args, **kw)
  mgr._write = delayed
  model = perturbed(4)
  t0 = time.perf_counter()
  assert mgr.save(1, model)
  assert time.perf_counter() - t0 < 0.25                 # returned while the writer is still asleep
  with torch.no_grad():
    for p in model.parameters():
      p.zero_()                                          # the snapshot was taken at save(): later changes do not leak in
  assert not mgr.save(2, model)                          # continuous policy: a write is in flight, skip
  mgr.close()
  restored = tiny()
  assert cm.CheckpointManager(str(tmp_path)).maybe_restore(restored)[0] == 1 and same(restored, perturbed(4))
