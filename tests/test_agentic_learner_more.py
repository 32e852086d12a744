"""Pieces of the agentic GRPO learner by themselves: turning collected trajectories into a training example
(padding, masks, advantages, degenerate groups, log-prob sources, KL on demand), sampler / trainer agreement and
truncated importance weights, the off-policy filter, prompt feeding, and the consumer's batching."""
import queue
import types

import numpy as np
import pytest
import torch

from tests.test_rl_grpo import ToyTokenizer, make_cluster, reward_len
from tunix_b200.common.datatypes import Mode
from tunix_b200.rl.agentic import agentic_grpo_learner as agl
from tunix_b200.rl.agentic.parser.chat_template_parser import parser as ctp


def learner(cluster=None, **cfg):
  cluster = cluster or make_cluster(max_steps=2)
  cfg.setdefault("num_generations", 2)
  cfg.setdefault("max_response_length", 8)
  return agl.GRPOLearner(rl_cluster=cluster, algo_config=agl.GRPOConfig(**cfg), reward_fns=[reward_len],
                         chat_parser=ctp.LlamaChatTemplateParser(ToyTokenizer()))


def trajectory(reply_tokens, reward_text, version=0, prompt=(5, 6, 7), lps=None, question="q"):
  n = len(reply_tokens)
  traj = {"conversation_text": [{"role": "user", "content": question}, {"role": "assistant", "content": reward_text}],
          "prompt_tokens": np.asarray(prompt), "conversation_tokens": np.asarray(reply_tokens),
          "conversation_masks": np.ones(n, np.int32), "old_logprobs": None if lps is None else np.asarray(lps, np.float32),
          "policy_version": version, "trajectory_reward": 0.0, "status": "SUCCEEDED",
          "original_input": {"prompts": [question], "answer": ["a"]}, "env_time": {"step_latency": [0.1, 0.3]},
          "reward_time": {"reward_latency": 0.01}}
  return types.SimpleNamespace(traj=traj)


def group(*pairs, **kw):
  return [trajectory(tokens, text, **kw) for tokens, text in pairs]


def test_trajectories_become_one_padded_example_with_group_relative_advantages():
  lr = learner()
  items = group(([10, 11, 12], "w1 w2 w3"), ([13], "w1"), lps=None)
  for it, lps in zip(items, ([-0.1, -0.2, -0.3], [-0.4])):
    it.traj["old_logprobs"] = np.asarray(lps, np.float32)
  (ex,) = lr._process_results(items, expected_step=0)
  assert ex.prompt_ids.shape == (2, 8) and ex.completion_ids.shape == (2, 8)
  assert ex.prompt_ids[0].tolist() == [0, 0, 0, 0, 0, 5, 6, 7] and ex.prompt_mask[0].tolist() == [False] * 5 + [True] * 3
  assert ex.completion_ids.tolist() == [[10, 11, 12, 0, 0, 0, 0, 0], [13, 0, 0, 0, 0, 0, 0, 0]]
  assert ex.completion_mask.sum(-1).tolist() == [3, 1]
  # reward_len = words / 8 -> rewards 3/8 and 1/8; the group's advantages are their z-scores (sample deviation)
  assert ex.advantages.tolist() == pytest.approx([2 ** -0.5, -(2 ** -0.5)], abs=1e-3)
  assert ex.old_per_token_logps[0, :3].tolist() == pytest.approx([-0.1, -0.2, -0.3]) and ex.old_per_token_logps[0, 3:].eq(0).all()
  assert ex.policy_version.tolist() == [0, 0] and ex.ref_per_token_logps is not None      # beta 0.04: the KL term needs them
  assert ex.ref_per_token_logps.shape == (2, 8) and ex.sampler_is_weights is None
  lr.rl_engine.close()


def test_long_replies_are_cut_and_counted_as_clipped():
  lr = learner()
  written = []
  lr.rl_engine.with_external_metrics_logger(lambda page: written.append(page.metrics))
  items = group((list(range(10, 22)), "w " * 12), ([30, 31], "w w"), lps=None)
  items[0].traj["old_logprobs"] = -np.ones(12, np.float32)
  items[1].traj["old_logprobs"] = -np.ones(2, np.float32)
  (ex,) = lr._process_results(items, expected_step=0)
  assert ex.completion_ids[0].tolist() == list(range(10, 18)) and ex.completion_mask[0].all()
  lr.rl_engine.global_steps = 1
  lr.rl_engine.buffer_metrics({})                               # moves the ledger past step 0
  page = written[0]
  assert page["generation/completions/clip_ratio"][0] == [0.5]
  assert page["generation/completions/max_raw_length"][0] == [8] and page["generation/completions/min_length"][0] == [2]
  assert page["trajectory/status/SUCCEEDED"][0] == [1.0]
  assert page["trajectory/env_time/step_latency/max"][0] == [pytest.approx(0.3)]
  lr.rl_engine.close()


def test_a_group_without_signal_can_be_masked_out():
  same = group(([10, 11], "w w"), ([12, 13], "w w"), lps=[-1.0, -1.0])
  kept = learner()
  (ex,) = kept._process_results(same, expected_step=0)
  assert ex.advantages.tolist() == [0.0, 0.0] and ex.completion_mask.sum() == 4
  masked = learner(degenerate_group_masking=True)
  (ex,) = masked._process_results(same, expected_step=0)
  assert ex.completion_mask.sum() == 0                          # nothing to learn from: no tokens, no denominator
  kept.rl_engine.close(); masked.rl_engine.close()


@pytest.mark.parametrize("beta, force, expect_ref", [(0.0, False, False), (0.0, True, True), (0.04, False, True)])
def test_reference_logps_are_computed_only_when_a_kl_is_wanted(beta, force, expect_ref):
  lr = learner(make_cluster(max_steps=1), beta=beta, force_compute_kl=force)          # the cluster has a reference model
  (ex,) = lr._process_results(group(([10], "w"), ([11, 12], "w w"), lps=[-1.0, -1.0][:1]), expected_step=0)
  assert (ex.ref_per_token_logps is not None) == expect_ref
  lr.rl_engine.close()


def test_trainer_logps_replace_rollout_logps_on_request():
  cluster = make_cluster(max_steps=1)
  cluster.sync_weights()                                         # the anchor policy scores old log-probs
  lr = learner(cluster, use_rollout_logps=False)
  items = group(([10, 11], "w w"), ([12], "w"), lps=[-9.0, -9.0])
  items[1].traj["old_logprobs"] = np.asarray([-9.0], np.float32)
  (ex,) = lr._process_results(items, expected_step=0)
  want = cluster.get_actor_per_token_logps(ex.prompt_ids, ex.completion_ids, 0, 2).cpu()
  torch.testing.assert_close(ex.old_per_token_logps, want)       # not the -9s the rollout reported
  lr.rl_engine.close()
  missing = group(([10], "w"), ([11], "w"))
  missing[0].traj["policy_version"] = None
  with pytest.raises(ValueError, match="policy_version is missing"):
    learner()._process_results(missing, expected_step=0)


def test_sampler_trainer_agreement_and_truncated_importance_weights():
  rollout = torch.log(torch.tensor([[0.5, 0.25, 0.9]]))
  trainer = torch.log(torch.tensor([[0.5, 0.75, 0.1]]))
  mask = torch.tensor([[1, 1, 0]])
  metrics, weights = agl.sampler_trainer_agreement(rollout, trainer, mask, None, 2.0)
  assert weights is None
  assert metrics["sampler_trainer/logp_diff_mean"][0] == pytest.approx(np.log(3) / 2, rel=1e-5)
  assert metrics["sampler_trainer/logp_diff_max"][0] == pytest.approx(np.log(3), rel=1e-5)   # the masked token is ignored
  assert metrics["sampler_trainer/prob_diff_mean"][0] == pytest.approx(0.25, rel=1e-5)
  metrics, weights = agl.sampler_trainer_agreement(rollout, trainer, mask, "token", 2.0)
  assert weights.tolist() == [[1.0, 2.0, 0.0]]                   # ratio 3 truncated at 2; nothing on masked tokens
  assert metrics["sampler_is/weight_mean"][0] == 1.5 and metrics["sampler_is/frac_clipped_at_threshold"][0] == 0.5
  assert not weights.requires_grad
  assert agl.sampler_trainer_agreement(None, trainer, mask, "token", 2.0) == ({}, None)
  perfect, _ = agl.sampler_trainer_agreement(rollout, rollout, torch.ones(1, 3), None, 2.0)
  assert perfect["sampler_trainer/probs_pearson_corr"][0] == pytest.approx(1.0, abs=1e-5)


def test_stale_examples_are_dropped_by_the_off_policy_window():
  lr = learner(off_policy_steps=1)
  make = lambda v: types.SimpleNamespace(policy_version=None if v is None else np.asarray([v, v]))
  lr.policy_version = 3
  kept = lr._filter_outdated_offpolicy_examples([make(3), make(2), make(1), make(-1), make(None)])
  assert [int(e.policy_version[0]) for e in kept] == [3, 2, -1]  # -1 marks examples that never expire
  assert lr._filter_outdated_offpolicy_examples([make(0)]) == []
  lr.rl_engine.close()


def test_prompt_feeding_stops_at_max_steps_partial_batches_and_the_end_of_data():
  lr = learner(make_cluster(max_steps=2))
  lr._full_batch_size = 2
  q = queue.Queue()
  full, partial = {"prompts": ["a", "b"]}, {"prompts": ["a"]}
  lr._put_prompts_to_queue(q, full)
  assert q.get_nowait() is full
  lr._put_prompts_to_queue(q, partial)
  assert q.get_nowait() is None                                  # a short batch ends the stream
  lr.rl_engine.global_steps = 2
  lr._put_prompts_to_queue(q, full)
  assert q.get_nowait() is None                                  # the step budget is spent
  lr.rl_engine.global_steps = 0
  lr._feed_next(iter([]), q)
  assert q.get_nowait() is None
  lr._feed_next(iter([full]), q)
  assert q.get_nowait() is full
  lr.rl_engine.close()


def test_the_consumer_batches_groups_flushes_the_tail_and_reraises_producer_errors():
  lr = learner()
  q = queue.Queue()
  for item in ("g1", "g2", "g3", None):
    q.put(item)
  assert list(lr._data_consumer_batch_generator(q, 2)) == [["g1", "g2"], ["g3"]]
  q.put("g1"); q.put(RuntimeError("rollout crashed"))
  gen = lr._data_consumer_batch_generator(q, 5)
  with pytest.raises(RuntimeError, match="rollout crashed"):
    next(gen)
  lr.rl_engine.close()
