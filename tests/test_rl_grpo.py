"""Toy end-to-end GRPO / DAPO / Dr.GRPO on CPU with the vanilla rollout engine, plus unit tests of
the RL math (advantages, KL, aggregation, packing)."""
import numpy as np
import pytest
import torch

from tunix_b200 import optim
from tunix_b200.common.configs import ClusterConfig, RLTrainingConfig, RolloutConfig
from tunix_b200.common.datatypes import Mode, Role
from tunix_b200.models.transformer import ModelConfig, Transformer
from tunix_b200.rl import algo_core, common, rl_cluster, utils as rl_utils
from tunix_b200.rl.grpo import dapo_learner, drgrpo_learner, grpo_learner


class ToyTokenizer:
  """Word-level tokenizer over a tiny fixed vocabulary."""

  def __init__(self, vocab=64):
    self.vocab = vocab

  def encode(self, s, **kw):
    return [3 + (sum(map(ord, w)) % (self.vocab - 3)) for w in s.split()]

  def decode(self, ids, **kw):
    return " ".join(f"w{int(i)}" for i in ids)

  def bos_id(self): return 1
  def eos_id(self): return 2
  def pad_id(self): return 0


def toy_model(seed=0, **kw):
  cfg = ModelConfig(num_layers=2, vocab_size=64, embed_dim=32, hidden_dim=64, num_heads=4, head_dim=8, num_kv_heads=2,
                    **kw)
  return Transformer(cfg).init_weights(seed=seed, scale=0.3)


def make_cluster(tmp_path=None, beta=0.04, ga=None, mini=None, micro=None, max_steps=4, lora=False, num_prompts=4,
                 return_logprobs=True, **tc_kw):
  actor = toy_model()
  reference = toy_model() if beta else None
  if lora:
    from tunix_b200.models import lora as lora_lib
    lora_lib.apply_lora_to_model(actor, rank=4, alpha=8.0)
  tc = RLTrainingConfig(actor_optimizer=optim.adamw(1e-2), eval_every_n_steps=100, max_steps=max_steps,
                        mini_batch_size=mini, train_micro_batch_size=micro, pbar_description=None,
                        checkpoint_root_directory=str(tmp_path) if tmp_path else None, **tc_kw)
  rc = RolloutConfig(max_tokens_to_generate=8, max_prompt_length=8, kv_cache_size=32, temperature=1.0, top_p=1.0,
                     seed=3, return_logprobs=return_logprobs)
  cc = ClusterConfig(role_to_mesh={Role.ACTOR: None, Role.REFERENCE: None, Role.ROLLOUT: None},
                     rollout_engine="vanilla", training_config=tc, rollout_config=rc)
  return rl_cluster.RLCluster(actor=actor, reference=reference, tokenizer=ToyTokenizer(), cluster_config=cc)


def prompts_ds(n_batches, batch=4):
  words = ["alpha", "beta", "gamma", "delta", "eps", "zeta", "eta", "theta"]
  for i in range(n_batches):
    yield {"prompts": [" ".join(words[(i + j + k) % 8] for k in range(3)) for j in range(batch)],
           "answer": [str(j) for j in range(batch)]}


def reward_len(prompts, completions, **kw):
  return [float(len(c.split())) / 8.0 for c in completions]


def reward_even(prompts, completions, answer=None, **kw):
  assert answer is not None and len(answer) == len(prompts)
  return [sum(1.0 for w in c.split() if int(w[1:]) % 2 == 0) / 8.0 for c in completions]


def test_grpo_end_to_end_trains_and_logs():
  cl = make_cluster()
  before = {n: p.clone() for n, p in cl.actor_trainer.model.named_parameters()}
  learner = grpo_learner.GRPOLearner(rl_cluster=cl, algo_config=grpo_learner.GRPOConfig(num_generations=2),
                                     reward_fns=[reward_len, reward_even])
  learner.train(prompts_ds(4))
  assert cl.actor_trainer.train_steps == 4
  assert cl.global_steps == 4
  changed = [n for n, p in cl.actor_trainer.model.named_parameters() if not torch.equal(p, before[n])]
  assert changed
  lg = cl._rl_metrics_logger
  assert lg.metric_exists("rewards", "score/mean", "train")
  assert lg.metric_exists("rewards", "reward_len", "train")
  assert lg.metric_exists("completions", "mean_length", "train")
  assert lg.metric_exists("", "kl", "train")
  assert len(lg.get_metric_history("", "loss", "train")) == 4


def test_grpo_micro_batching_is_equivalent():
  """mini=4 with micro=2 (2 accumulation steps) must reach the same weights as micro=4."""
  res = []
  for micro in (4, 2):
    torch.manual_seed(0)
    cl = make_cluster(mini=4, micro=micro, max_steps=2, beta=0.0, rollout_micro_batch_size=4,
                      compute_logps_micro_batch_size=4)
    learner = grpo_learner.GRPOLearner(rl_cluster=cl, algo_config=grpo_learner.GRPOConfig(
        num_generations=2, beta=0.0, loss_agg_mode="token-mean"), reward_fns=reward_len)
    learner.train(prompts_ds(2))
    res.append({n: p.detach().clone() for n, p in cl.actor_trainer.model.named_parameters()})
  for n in res[0]:
    torch.testing.assert_close(res[0][n], res[1][n], rtol=2e-4, atol=2e-5, msg=n)


def test_grpo_multi_iteration_and_gspo():
  cl = make_cluster(max_steps=4)
  cfg = grpo_learner.GRPOConfig(num_generations=2, num_iterations=2, loss_algo="gspo-token")
  learner = grpo_learner.GRPOLearner(rl_cluster=cl, algo_config=cfg, reward_fns=reward_len)
  learner.train(prompts_ds(2))
  assert cl.actor_trainer.train_steps == 4      # 2 batches x mu=2


def test_grpo_without_rollout_logprobs_recomputes_on_trainer():
  cl = make_cluster(return_logprobs=False, max_steps=2)
  cl.sync_weights()                # creates the anchor snapshot
  cfg = grpo_learner.GRPOConfig(num_generations=2, use_rollout_logps=False)
  learner = grpo_learner.GRPOLearner(rl_cluster=cl, algo_config=cfg, reward_fns=reward_len)
  learner.train(prompts_ds(2))
  assert cl.actor_trainer.train_steps == 2


def test_producer_exception_propagates():
  cl = make_cluster()

  def bad_reward(prompts, completions, **kw):
    raise RuntimeError("boom")
  learner = grpo_learner.GRPOLearner(rl_cluster=cl, algo_config=grpo_learner.GRPOConfig(num_generations=2),
                                     reward_fns=bad_reward)
  with pytest.raises(RuntimeError, match="boom"):
    learner.train(prompts_ds(2))


def test_dapo_and_drgrpo():
  cl = make_cluster(beta=0.0, max_steps=2)
  cfg = dapo_learner.DAPOConfig(num_generations=2, overlong_buffer={
      "enable": True, "overlong_buffer_length": 4, "overlong_buffer_penalty": 1.0, "max_response_length": 8})
  dapo_learner.DAPOLearner(rl_cluster=cl, algo_config=cfg, reward_fns=reward_len).train(prompts_ds(2))
  assert cl.actor_trainer.train_steps == 2
  with pytest.raises(ValueError):
    dapo_learner.DAPOConfig(num_generations=2, beta=0.1)
  cl2 = make_cluster(beta=0.0, max_steps=2)
  cfg2 = drgrpo_learner.DrGRPOConfig(num_generations=2, beta=0.0)
  assert cfg2.advantage_estimator == "drgrpo" and cfg2.loss_agg_mode == "sequence-mean-token-scale"
  drgrpo_learner.DrGRPOLearner(rl_cluster=cl2, algo_config=cfg2, reward_fns=reward_len).train(prompts_ds(2))
  assert cl2.actor_trainer.train_steps == 2


def test_resume_from_checkpoint(tmp_path):
  cl = make_cluster(tmp_path=tmp_path, max_steps=2)
  grpo_learner.GRPOLearner(rl_cluster=cl, algo_config=grpo_learner.GRPOConfig(num_generations=2),
                           reward_fns=reward_len).train(prompts_ds(4))
  w = {n: p.detach().clone() for n, p in cl.actor_trainer.model.named_parameters()}
  cl2 = make_cluster(tmp_path=tmp_path, max_steps=4)
  assert cl2.actor_trainer.train_steps == 2
  for n, p in cl2.actor_trainer.model.named_parameters():
    torch.testing.assert_close(p, w[n], msg=n)
  learner = grpo_learner.GRPOLearner(rl_cluster=cl2, algo_config=grpo_learner.GRPOConfig(num_generations=2),
                                     reward_fns=reward_len)
  assert cl2.global_steps == 2
  learner.train(prompts_ds(4))
  assert cl2.actor_trainer.train_steps == 4


def test_lora_actor_shares_backbone_with_reference_and_syncs_only_lora():
  cl = make_cluster(lora=True, max_steps=2)
  learner = grpo_learner.GRPOLearner(rl_cluster=cl, algo_config=grpo_learner.GRPOConfig(num_generations=2),
                                     reward_fns=reward_len)
  learner.train(prompts_ds(2))
  assert cl.actor_trainer.train_steps == 2


def test_sequence_packing_path():
  cl = make_cluster(max_steps=2, beta=0.0, max_seq_token_per_tpu=64)
  cfg = grpo_learner.GRPOConfig(num_generations=2, beta=0.0, loss_agg_mode="token-mean")
  grpo_learner.GRPOLearner(rl_cluster=cl, algo_config=cfg, reward_fns=reward_len).train(prompts_ds(2))
  assert cl.actor_trainer.train_steps == 2


# ---- unit tests -----------------------------------------------------------------------------
def test_advantage_estimators():
  r = np.array([1.0, 2.0, 3.0, 4.0, 2.0, 2.0, 2.0, 2.0])
  a = algo_core.compute_advantages(r, 4)
  g = r[:4]
  np.testing.assert_allclose(a[:4], (g - g.mean()) / (g.std(ddof=1) + 1e-6), rtol=1e-5)
  np.testing.assert_allclose(a[4:], 0.0, atol=1e-6)
  np.testing.assert_allclose(algo_core.compute_drgrpo_advantages(r, 4)[:4], g - g.mean(), rtol=1e-6)
  np.testing.assert_allclose(algo_core.compute_rloo_advantages(r, 4)[:4], g - (g.sum() - g) / 3, rtol=1e-6)


def test_gae_matches_reference_recursion():
  torch.manual_seed(0)
  r, v = torch.rand(3, 6), torch.rand(3, 6)
  m = torch.tensor([[1, 1, 1, 1, 0, 0], [1, 1, 1, 1, 1, 1], [1, 1, 0, 0, 0, 0]]).float()
  adv, ret = algo_core.compute_gae_advantages(r, v, m, 0.99, 0.95)
  # independent per-row recursion over valid steps only
  raw = torch.zeros_like(v)
  for b in range(3):
    L = int(m[b].sum())
    gae, nv = 0.0, 0.0
    for t in range(L - 1, -1, -1):
      delta = r[b, t] + 0.99 * nv - v[b, t]
      gae = delta + 0.99 * 0.95 * gae
      raw[b, t] = gae
      nv = v[b, t]
  torch.testing.assert_close((ret - v) * m, raw * m, rtol=1e-5, atol=1e-6)
  w = (adv * m).sum() / m.sum()
  assert abs(w.item()) < 1e-5


def test_kl_estimators_and_clamp():
  lp, ref = torch.tensor([-1.0, -2.0]), torch.tensor([-1.5, -1.0])
  torch.testing.assert_close(common.compute_kl_divergence(lp, ref, "kl"), lp - ref)
  torch.testing.assert_close(common.compute_kl_divergence(lp, ref, "mse_kl"), 0.5 * (lp - ref) ** 2)
  d = ref - lp
  torch.testing.assert_close(common.compute_kl_divergence(lp, ref, "low_var_kl"), d.exp() - d - 1)
  assert common.compute_kl_divergence(lp, ref, "kl", clamp_value=0.1).abs().max() <= 0.1 + 1e-7
  with pytest.raises(ValueError):
    common.compute_kl_divergence(lp, ref, "nope")


@pytest.mark.parametrize("mode", ["token-mean", "sequence-mean-token-mean", "sequence-mean-token-scale",
                                  "seq-mean-token-sum", "sequence-mean-token-sum-norm"])
def test_reduced_equals_unreduced_and_packing_invariance(mode):
  torch.manual_seed(1)
  B, T = 4, 6
  loss = torch.randn(B, T)
  lens = [6, 3, 2, 4]
  mask = torch.stack([(torch.arange(T) < n).float() for n in lens])
  kw = {"norm": 5.0} if mode in ("sequence-mean-token-scale", "sequence-mean-token-sum-norm") else {}
  wm = common.aggregate_loss(loss, mask, mode, **kw)
  torch.testing.assert_close(wm.compute(), common.reduced_loss_agg(loss, mask, mode, **kw), rtol=1e-5, atol=1e-6)
  # the same sequences packed into two rows give the same value
  row0 = torch.cat([loss[0, :6], loss[1, :3]])
  row1 = torch.cat([loss[3, :4], loss[2, :2], torch.zeros(3)])
  packed = torch.stack([row0, row1])
  pmask = torch.stack([torch.ones(9), torch.cat([torch.ones(6), torch.zeros(3)])])
  seg = torch.stack([torch.tensor([1] * 6 + [2] * 3), torch.tensor([1] * 4 + [2] * 2 + [0] * 3)])
  if mode == "sequence-mean-token-sum-norm":
    kw = {"norm": 5.0}
  wp = common.aggregate_loss(packed, pmask, mode, segment_ids=seg, num_segments=4, **kw)
  if mode != "sequence-mean-token-sum-norm":
    torch.testing.assert_close(wp.compute(), wm.compute(), rtol=1e-5, atol=1e-6)
  torch.testing.assert_close(wp.compute(), common.reduced_loss_agg(packed, pmask, mode, segment_ids=seg,
                                                                   num_segments=4, **kw), rtol=1e-5, atol=1e-6)


def test_completion_mask_and_padding():
  ids = torch.tensor([[5, 6, 2, 0, 0], [5, 6, 7, 8, 9]])
  assert common.make_completion_mask(ids, eos_tok=2).tolist() == [[1, 1, 1, 0, 0], [1, 1, 1, 1, 1]]
  assert common.np_make_completion_mask(ids.numpy(), eos_tok=2).tolist() == [[1, 1, 1, 0, 0], [1, 1, 1, 1, 1]]
  assert common.pad_to_length(np.array([1, 2]), 4, 9, left=True).tolist() == [9, 9, 1, 2]
  assert common.pad_to_length(torch.tensor([1, 2]), 1).tolist() == [1, 2]


def test_pack_sequences_ffd_and_update_boundaries():
  def ex(lens_p, lens_c):
    B = len(lens_p)
    P, C = 4, 6
    p = torch.zeros(B, P, dtype=torch.long)
    pm = torch.zeros(B, P, dtype=torch.int32)
    c = torch.zeros(B, C, dtype=torch.long)
    cm = torch.zeros(B, C, dtype=torch.int32)
    for i, (a, b) in enumerate(zip(lens_p, lens_c)):
      p[i, P - a:] = 7
      pm[i, P - a:] = 1
      c[i, :b] = 9
      cm[i, :b] = 1
    return common.TrainExample(prompt_ids=p, prompt_mask=pm, completion_ids=c, completion_mask=cm,
                               advantages=torch.arange(B).float(), ref_per_token_logps=None,
                               old_per_token_logps=torch.ones(B, C))
  stream = [[ex([2, 3], [4, 2])], [ex([4, 1], [6, 1])]]
  out = list(rl_utils.pack_sequences(iter(stream), max_token_budget=12, sequences_per_update=4, pack_size=1))
  flags = [bool(o[0].is_update_step[0]) for o in out]
  assert flags[-1] and not any(flags[:-1])
  total = sum(int((o[0].segment_ids > 0).sum()) for o in out)
  assert total == (2 + 4) + (3 + 2) + (4 + 6) + (1 + 1)
  for o in out:
    e = o[0]
    assert e.completion_ids.shape == (1, 12) and e.num_segments == 13
    seg = e.segment_ids[0]
    for s in seg.unique():
      if s == 0:
        continue
      pos = e.segment_positions[0][seg == s]
      assert pos.tolist() == list(range(len(pos)))
    assert e.old_per_token_logps is not None
  with pytest.raises(ValueError, match="exceeding"):
    list(rl_utils.pack_sequences(iter([[ex([4], [6])]]), max_token_budget=8, sequences_per_update=1))
  with pytest.raises(ValueError, match="mid-mini-batch"):
    list(rl_utils.pack_sequences(iter([[ex([1], [1])]]), max_token_budget=8, sequences_per_update=2))


def test_ppo_end_to_end_with_critic():
  from tunix_b200.rl.ppo import ppo_learner
  actor, reference = toy_model(), toy_model()
  critic = rl_utils.create_critic_model(toy_model(seed=1))
  tc = RLTrainingConfig(actor_optimizer=optim.adamw(1e-2), critic_optimizer=optim.adamw(1e-2), eval_every_n_steps=100,
                        max_steps=3, pbar_description=None)
  rc = RolloutConfig(max_tokens_to_generate=8, max_prompt_length=8, kv_cache_size=32, temperature=1.0, top_p=1.0, seed=3)
  cc = ClusterConfig(role_to_mesh={Role.ACTOR: None, Role.REFERENCE: None, Role.ROLLOUT: None, Role.CRITIC: None},
                     rollout_engine="vanilla", training_config=tc, rollout_config=rc)
  cl = rl_cluster.RLCluster(actor=actor, reference=reference, critic=critic, tokenizer=ToyTokenizer(), cluster_config=cc)
  before = {n: p.clone() for n, p in cl.critic_trainer.model.named_parameters()}
  cfg = ppo_learner.PPOConfig(entropy_coef=0.01, epsilon_c=3.0)
  assert cfg.epsilon_low == cfg.epsilon_high == 0.2
  with pytest.raises(ValueError):
    ppo_learner.PPOLearner(rl_cluster=cl, algo_config=cfg, reward_fns=None)
  ppo_learner.PPOLearner(rl_cluster=cl, algo_config=cfg, reward_fns=reward_len).train(prompts_ds(3))
  assert cl.actor_trainer.train_steps == 3 and cl.critic_trainer.train_steps == 3
  assert any(not torch.equal(p, before[n]) for n, p in cl.critic_trainer.model.named_parameters())
  lg = cl._rl_metrics_logger
  assert lg.metric_exists("advantages", "returns/mean", "train")
  assert lg.metric_exists("", "vpred_mean", "train")


def test_engine_with_its_own_weight_copy_is_synced_every_step():
  """An engine that keeps a private copy (vLLM) reports the actor as its model; the learner must still push the
  parameters after every optimizer step (`holds_own_weights`)."""
  from tunix_b200.rl.rollout import base_rollout, vanilla_rollout

  class PrivateCopyRollout(vanilla_rollout.VanillaRollout):
    holds_own_weights = True
    pushes = 0

    def __init__(self, rollout_actor, tokenizer, mesh, rollout_config):
      mc = rollout_actor.config
      super().__init__(rollout_actor, tokenizer, base_rollout.CacheConfig(
          cache_size=rollout_config.kv_cache_size, num_layers=mc.num_layers, num_kv_heads=mc.num_kv_heads,
          head_dim=mc.head_dim))

    def update_params(self, params, filter_types=None):
      type(self).pushes += 1

  import dataclasses
  cc = dataclasses.replace(make_cluster(max_steps=3).cluster_config, rollout_engine=PrivateCopyRollout)
  cl2 = rl_cluster.RLCluster(actor=toy_model(), reference=toy_model(), tokenizer=ToyTokenizer(), cluster_config=cc)
  learner = grpo_learner.GRPOLearner(rl_cluster=cl2, algo_config=grpo_learner.GRPOConfig(num_generations=2),
                                     reward_fns=reward_len)
  assert learner.should_sync_weights
  learner.train(prompts_ds(3))
  assert PrivateCopyRollout.pushes == 3 and cl2.global_steps == 3
