"""`RLCluster` / `RLEngine`: configuration errors, engine selection (names, user classes), per-mode rollout
configs, chat templates, micro-batched generation, log-prob services of the roles, the step ledger of RL metrics,
role training entry points, and weight sync bookkeeping."""
import dataclasses

import numpy as np
import pytest
import torch

from tunix_b200 import optim
from tunix_b200.common.configs import ClusterConfig, RLTrainingConfig, RolloutConfig
from tunix_b200.common.datatypes import Mode, Role
from tunix_b200.rl import common, rl_cluster
from tunix_b200.rl.rollout import base_rollout, vanilla_rollout
from tests.test_rl_grpo import ToyTokenizer, make_cluster, toy_model


def config(**kw):
  return dataclasses.replace(make_cluster().cluster_config, **kw)


def cluster(cc, **kw):
  kw.setdefault("actor", toy_model())
  kw.setdefault("reference", toy_model())
  kw.setdefault("tokenizer", ToyTokenizer())
  return rl_cluster.RLCluster(cluster_config=cc, **kw)


def test_alias_and_configuration_errors():
  assert rl_cluster.RLCluster is rl_cluster.RLEngine
  with pytest.raises(ValueError, match="rollout_config` cannot be None"):
    cluster(config(rollout_config=None))
  rc = make_cluster().cluster_config.rollout_config
  with pytest.raises(ValueError, match="missing a train config"):
    cluster(config(rollout_config={Mode.EVAL: rc}))
  with pytest.raises(NotImplementedError, match="not supported"):
    cluster(config(rollout_engine="teletype"))
  class Configless(torch.nn.Module):
    def __init__(self):
      super().__init__()
      self.w = torch.nn.Parameter(torch.zeros(1))
  with pytest.raises(ValueError, match="needs a model with a `config`"):
    cluster(config(), actor=Configless(), reference=None)


def test_rollout_config_per_mode_and_generation_budget_override():
  train = make_cluster().cluster_config.rollout_config
  evaluation = dataclasses.replace(train, max_tokens_to_generate=3, temperature=0.0)
  cl = cluster(config(rollout_config={Mode.TRAIN: train, Mode.EVAL: evaluation}))
  assert cl.get_rollout_config(Mode.TRAIN) is train and cl.get_rollout_config(Mode.EVAL) is evaluation
  prompts = ["alpha beta", "gamma"]
  assert max(len(t) for t in cl.generate(prompts, mode=Mode.TRAIN).tokens) <= 8
  assert max(len(t) for t in cl.generate(prompts, mode=Mode.EVAL).tokens) <= 3
  assert max(len(t) for t in cl.generate(prompts, mode=Mode.TRAIN, max_generation_steps=2).tokens) <= 2
  with pytest.raises(ValueError, match="empty list of prompts"):
    cl.generate([])
  cl.close()


def test_generation_in_micro_batches_joins_outputs_in_order():
  cl = cluster(config(rollout_config=dataclasses.replace(make_cluster().cluster_config.rollout_config, temperature=0.0,
                                                         top_p=None)))
  prompts = ["alpha beta", "gamma", "delta eps zeta", "eta", "theta iota"]
  whole = cl.generate(prompts)
  pieces = cl.generate(prompts, micro_batch_size=2)
  assert len(pieces.text) == 5 and pieces.left_padded_prompt_tokens.shape[0] == 5
  assert [t.tolist() for t in pieces.tokens] == [t.tolist() for t in whole.tokens]
  assert pieces.logprobs is not None and len(pieces.logprobs) == 5
  cl.close()


def test_chat_templates_go_through_the_tokenizer():
  class ChatTokenizer(ToyTokenizer):
    rendered = []
    def apply_chat_template(self, chat, add_generation_prompt=True, tokenize=False, **kw):
      text = " ".join(m["content"] for m in chat) + (" assistant" if add_generation_prompt else "")
      self.rendered.append(text)
      return text
  cl = cluster(config(), tokenizer=ChatTokenizer())
  out = cl.generate([[{"role": "user", "content": "alpha beta"}]], apply_chat_template=True)
  assert ChatTokenizer.rendered == ["alpha beta assistant"] and len(out.tokens) == 1
  cl.close()


def test_a_user_defined_engine_class_is_instantiated_with_the_documented_arguments():
  seen = {}

  class Mine(vanilla_rollout.VanillaRollout):
    def __init__(self, rollout_actor, tokenizer, mesh, rollout_config):
      seen.update(actor=rollout_actor, mesh=mesh, rc=rollout_config)
      mc = rollout_actor.config
      super().__init__(rollout_actor, tokenizer, base_rollout.CacheConfig(
          cache_size=rollout_config.kv_cache_size, num_layers=mc.num_layers, num_kv_heads=mc.num_kv_heads,
          head_dim=mc.head_dim))
  cc = config(rollout_engine=Mine)
  cl = cluster(cc)
  assert isinstance(cl.rollout, Mine) and seen["rc"] is cc.rollout_config and seen["mesh"] is None
  # a private engine gets its own copy of the actor, so training the actor needs a sync to reach it
  assert seen["actor"] is not cl.actor_trainer.model
  assert len(cl.generate(["alpha"]).tokens) == 1
  cl.close()


def test_log_prob_services_of_the_roles_agree_with_direct_scoring():
  cl = cluster(config())
  g = torch.Generator().manual_seed(0)
  prompt, completion = torch.randint(3, 64, (3, 5), generator=g), torch.randint(3, 64, (3, 4), generator=g)
  direct = common.compute_per_token_logps(cl.actor_trainer.model, prompt, completion, 0, 2)
  torch.testing.assert_close(cl.get_old_per_token_logps(prompt, completion), direct)
  torch.testing.assert_close(cl.get_old_per_token_logps(prompt, completion, micro_batch_size=2), direct)
  ref = cl.get_ref_per_token_logps(prompt, completion, 0, 2, micro_batch_size=1)
  torch.testing.assert_close(ref, common.compute_per_token_logps(cl.reference, prompt, completion, 0, 2))
  torch.testing.assert_close(cl.per_token_logps(Role.REFERENCE, prompt, completion, 0, 2), ref)
  with pytest.raises(ValueError, match="empty batch"):
    cl.get_old_per_token_logps(prompt[:0], completion[:0])
  cl.close()


def test_anchor_policy_scores_with_the_weights_of_the_last_sync():
  cl = cluster(config())
  g = torch.Generator().manual_seed(1)
  prompt, completion = torch.randint(3, 64, (2, 5), generator=g), torch.randint(3, 64, (2, 4), generator=g)
  with pytest.raises(ValueError, match="sync_weights` first"):
    cl.get_actor_per_token_logps(prompt, completion, 0, 2)
  at_sync = common.compute_per_token_logps(cl.actor_trainer.model, prompt, completion, 0, 2)
  cl.sync_weights()
  assert cl.global_steps == 1
  with torch.no_grad():
    for p in cl.actor_trainer.model.parameters():
      p.add_(0.05)                                                      # the actor trains on
  moved = common.compute_per_token_logps(cl.actor_trainer.model, prompt, completion, 0, 2)
  anchored = cl.get_actor_per_token_logps(prompt, completion, 0, 2)
  torch.testing.assert_close(anchored, at_sync, rtol=1e-5, atol=1e-6)
  assert not torch.allclose(anchored, moved)
  torch.testing.assert_close(common.compute_per_token_logps(cl.actor_trainer.model, prompt, completion, 0, 2), moved)
  cl.close()


def test_metrics_ledger_writes_a_step_once_the_run_has_left_it():
  cl = cluster(config())
  written = []
  cl.with_external_metrics_logger(lambda page: written.append((page.global_steps, dict(page.metrics))))
  cl.buffer_metrics({"rewards/mean": (1.0, np.mean), "completions/text": ("hello", None)})
  cl.buffer_metrics({"rewards/mean": (3.0, np.mean)})
  assert written == []                                                    # step 0 is still current
  cl.buffer_metrics_async({"rollout/lag": (5.0, np.max)}, step=1)         # a producer that runs ahead
  cl.global_steps = 1
  cl.buffer_metrics({"rewards/mean": (10.0, np.mean)})
  assert [s for s, _ in written] == [0] and written[0][1]["rewards/mean"][0] == [1.0, 3.0]
  lg = cl._rl_metrics_logger
  assert lg.get_metric_history("rewards", "mean", "train").tolist() == [2.0]
  assert not lg.metric_exists("completions", "text", "train")             # strings are logged as text, not as scalars
  cl.global_steps = 2
  cl.buffer_metrics({}, mode=Mode.EVAL)
  assert [s for s, _ in written] == [0, 1]
  assert set(written[1][1]) == {"rollout/lag", "rewards/mean"}            # both writers of step 1 share one page
  cl.close()
  assert [s for s, _ in written] == [0, 1, 2]                             # close flushes what is left


def test_role_training_entry_points():
  cl = cluster(config())
  with pytest.raises(ValueError, match="Unsupported role for train"):
    cl.train(Role.REFERENCE, [], None)
  assert cl.eval_actor(None) is None
  assert isinstance(cl.rollout, base_rollout.BaseRollout) and cl.inference_worker is not None
  assert cl.weight_sync_ms() is None                                      # the vanilla engine does not time syncs
  cl.close()
