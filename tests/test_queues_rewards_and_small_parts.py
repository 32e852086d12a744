"""Trajectory queue (grouping, staleness, custom grouping and filters, leftovers, poisoning, ledger), the rollout
collector's single-call path, reward managers, algorithm configuration, the progress bar and the TFLOP estimate."""
import asyncio
import dataclasses
import logging

import numpy as np
import pytest

from tunix_b200.experimental.common import datatypes, test_utils
from tunix_b200.experimental.queue_manager import trajectory_queue_manager as tqm
from tunix_b200.experimental.rollout import collector
from tunix_b200.rl import algorithm_config, reward_manager
from tunix_b200.sft import metrics_logger as ml, progress_bar, system_metrics_calculator as smc


def item(group, idx, version=0):
  return datatypes.TrajectoryItem(pair_index=idx, group_id=group, start_step=0, traj={}, policy_version=version)


# ---- trajectory queue ---------------------------------------------------------------------------------
def test_items_are_grouped_by_group_id_and_released_as_whole_groups():
  async def go():
    q = tqm.TrajectoryQueueManager.create(group_size=2)
    for g, i in [("a", 0), ("b", 0), ("b", 1), ("a", 1), ("c", 0)]:
      await q.put(item(g, i))
    first, second = await q.get_group(), await q.get_group()
    assert [(x.group_id, x.pair_index) for x in first] == [("b", 0), ("b", 1)]      # b completed first
    assert [x.group_id for x in second] == ["a", "a"]
    await q.prepare_clear()
    assert await q.get_group() == []                                               # c never completed
    seen = [g async for g in q]
    assert seen == []
  asyncio.run(go())


def test_default_key_falls_back_from_group_id_to_prompt_id_to_identity():
  class P:
    def __init__(self, group_id=None, prompt_id=""):
      self.group_id, self.prompt_id = group_id, prompt_id
  assert tqm.default_group_key(P(group_id=0)) == 0                                  # 0 is a valid group id
  assert tqm.default_group_key(P(prompt_id="p7")) == "p7"
  x = P()
  assert tqm.default_group_key(x) == id(x) != tqm.default_group_key(P())


def test_stale_members_are_dropped_when_the_group_completes_and_reported():
  async def go():
    version = [5]
    q = tqm.TrajectoryQueueManager.create(group_size=3, max_staleness=1, current_policy_version=lambda: version[0],
                                          filter_fn=lambda g: [x for x in g if x.pair_index != 2])
    for idx, v in enumerate([5, 3, 4]):
      await q.put(item("g", idx, version=v))
    got = await q.get_group()
    assert [(x.pair_index, x.policy_version) for x in got] == [(0, 5)]             # v3 is stale, index 2 is filtered
    rejected = await q.get_filtered_groups()
    assert sorted(x.pair_index for x in rejected[0]) == [1, 2] and await q.get_filtered_groups() == []
  asyncio.run(go())


def test_custom_grouping_and_batches_that_cut_through_groups():
  async def go():
    def pairs_of_equal_parity(buckets, it):
      bucket = buckets[it.pair_index % 2]
      bucket.append(it)
      return buckets.pop(it.pair_index % 2) if len(bucket) == 2 else None
    q = tqm.TrajectoryQueueManager(group_fn=pairs_of_equal_parity)
    for i in [0, 1, 3, 2, 4]:
      await q.put(item("g", i))
    assert [x.pair_index for x in await q.get_batch(num_groups=2)] == [1, 3, 0, 2]
    q2 = tqm.TrajectoryQueueManager.create(group_size=3)
    for g in "ab":
      for i in range(3):
        await q2.put(item(g, i))
    head = await q2.get_batch(batch_size=4)
    assert [(x.group_id, x.pair_index) for x in head] == [("a", 0), ("a", 1), ("a", 2), ("b", 0)]
    assert [(x.group_id, x.pair_index) for x in await q2.get_group()] == [("b", 1), ("b", 2)]   # the rest of b
    await q2.put(item("c", 0))
    await q2.prepare_clear()
    assert await q2.get_batch(num_groups=3) == [] and await q2.get_batch() == []
  asyncio.run(go())


def test_a_producer_failure_poisons_the_queue_until_it_is_cleared_and_the_ledger_counts_items():
  async def go():
    q = tqm.TrajectoryQueueManager.create(group_size=1)
    waiting = asyncio.create_task(q.get_group())
    await asyncio.sleep(0.01)
    await q.put_exception(RuntimeError("rollout worker died"))
    with pytest.raises(RuntimeError, match="rollout worker died"):
      await waiting
    with pytest.raises(RuntimeError, match="rollout worker died"):
      await q.put(item("g", 0))
    await q.clear()
    await q.put(item("g", 0))
    group = await q.get_group()
    q.commit(7, [group, group])
    assert q.committed_items(7) == 2 and q.committed_items(8) == 0
  asyncio.run(go())


# ---- collector ------------------------------------------------------------------------------------------
def test_a_request_without_environment_is_one_sampling_call():
  async def go():
    sampler = test_utils.MockSampler(reply_fn=lambda prompt, v: "seen:" + prompt[-12:])
    parser = test_utils.MockChatParser()
    tok = sampler.tokenizer

    def request(prompt, **meta):
      return datatypes.RolloutRequest(request_id="r1", prompt=prompt, prompt_id="p1", target_policy_version=4,
                                      generation_kwargs={"max_tokens": 64}, metadata=meta)
    chat = await collector.TrajectoryCollectorEngine("t", request([{"role": "user", "content": "hello"}], tag="x"),
                                                     sampler, chat_parser=parser).run()
    assert chat.status == "SUCCEEDED" and chat.request_id == "r1" and chat.prompt_id == "p1" and chat.metadata == {"tag": "x"}
    assert chat.policy_version == 4 and len(chat.segments) == 1 and chat.segments[0].source == "assistant"
    assert tok.decode(chat.segments[0].tokens.tolist()).startswith("seen:")
    assert chat.segments[0].loss_mask.all() and np.allclose(chat.segments[0].logps, -0.5)
    templated = tok.decode(chat.prompt_tokens.tolist())
    assert "hello" in templated and templated != "hello"                            # the chat template was applied
    text = await collector.TrajectoryCollectorEngine("t", request("plain words"), sampler, chat_parser=parser).run()
    assert "plain words" in tok.decode(text.prompt_tokens.tolist())                  # a string becomes a user turn
    raw = await collector.TrajectoryCollectorEngine("t", request("plain words"), sampler).run()
    assert tok.decode(raw.prompt_tokens.tolist()) == "plain words"                   # no parser: passed through
    assert sampler.served == 3
  asyncio.run(go())


def test_failures_and_cancellations_come_back_in_band():
  async def go():
    class Broken(test_utils.MockSampler):
      async def sample(self, reqs, **kw):
        raise ConnectionError("engine unreachable")
    req = datatypes.RolloutRequest(request_id="r", prompt="x", prompt_id="p", metadata={"k": 1})
    failed = await collector.TrajectoryCollectorEngine("t", req, Broken()).run()
    assert failed.status == "FAILED" and failed.error.error_type == "ConnectionError" and failed.metadata == {"k": 1}
    assert "engine unreachable" in failed.error.message and "Traceback" in failed.error.traceback

    class Refusing(test_utils.MockSampler):
      async def sample(self, reqs, **kw):
        from tunix_b200.experimental.rollout import sampler as s
        return [s.SamplingResponse(error=datatypes.ErrorInfo(error_type="OOM", message="kv cache full"))]
    refused = await collector.TrajectoryCollectorEngine("t", req, Refusing()).run()
    assert refused.status == "FAILED" and "OOM: kv cache full" in refused.error.message

    class Slow(test_utils.MockSampler):
      async def sample(self, reqs, **kw):
        raise asyncio.CancelledError()
    cancelled = await collector.TrajectoryCollectorEngine("t", req, Slow()).run()
    assert cancelled.status == "CANCELLED" and cancelled.error.retryable
  asyncio.run(go())


# ---- reward managers ------------------------------------------------------------------------------------
def length(prompts, completions, **kw):
  return [float(len(c)) for c in completions]


def with_answer(prompts, completions, answer, bonus, **kw):
  return [bonus if a in c else 0.0 for c, a in zip(completions, answer)]


def undefined(prompts, completions, **kw):
  return [float("nan")] * len(completions)


@dataclasses.dataclass(kw_only=True)
class Cfg(algorithm_config.AlgorithmConfig):
  bonus: float = 2.0
  answer: str = "from config"


PROMPTS, DONE = ["p1", "p2", "p3"], ["a", "bb 4", "ccc"]


def test_rewards_are_summed_over_functions_with_columns_and_config_fields_passed_by_name():
  m = reward_manager.SequenceRewardManager([length, with_answer], Cfg())
  out = m(PROMPTS, DONE, answer=["x", "4", "c"])            # the batch column wins over the config field of that name
  assert out["rewards"].tolist() == [1.0, 6.0, 5.0]
  lm = out["log_metrics"]
  assert lm["rewards/length"][0].tolist() == [1.0, 4.0, 3.0] and lm["rewards/with_answer"][0].tolist() == [0.0, 2.0, 2.0]
  assert lm["rewards/sum"][0].tolist() == [1.0, 6.0, 5.0] and lm["rewards/mean"][0].tolist() == [0.5, 3.0, 2.5]
  assert lm["rewards/min"][0].tolist() == [0.0, 2.0, 2.0] and lm["rewards/max"][1] is np.max
  assert lm["prompts"] == (PROMPTS, None) and lm["completions"] == (DONE, None)
  single = reward_manager.SequenceRewardManager(length, Cfg())               # a bare function is accepted
  assert single(PROMPTS, DONE)["rewards"].tolist() == [1.0, 4.0, 3.0]
  from tunix_b200.rl import function_registry
  assert function_registry.get_reward_manager("sequence-level") is reward_manager.SequenceRewardManager


def test_nan_rewards_count_as_zero_in_the_sum_and_stay_visible_in_the_log():
  out = reward_manager.SequenceRewardManager([length, undefined], Cfg())(PROMPTS, DONE)
  assert out["rewards"].tolist() == [1.0, 4.0, 3.0]
  assert np.isnan(out["log_metrics"]["rewards/undefined"][0]).all()
  assert out["log_metrics"]["rewards/sum"][0].tolist() == [1.0, 4.0, 3.0]


def test_reward_function_mistakes_are_named():
  with pytest.raises(ValueError, match="cannot be empty"):
    reward_manager.SequenceRewardManager([], Cfg())
  nothing = reward_manager.SequenceRewardManager([lambda prompts, completions, **kw: None], Cfg())
  with pytest.raises(RuntimeError, match="Failed to obtain result.*Result is None"):
    nothing(PROMPTS, DONE)
  too_many = reward_manager.SequenceRewardManager([lambda prompts, completions, **kw: [1.0] * 4], Cfg())
  with pytest.raises(RuntimeError, match="Length mismatch"):
    too_many(PROMPTS, DONE)


def test_the_agentic_manager_adds_environment_rewards_and_works_without_functions():
  env_only = reward_manager.AgenticSequenceRewardManager(None, Cfg())
  out = env_only(PROMPTS, DONE, trajectory_rewards=[1.0, 0.0, 0.5])
  assert out["rewards"].tolist() == [1.0, 0.0, 0.5] and out["log_metrics"]["trajectory_rewards/mean"][0] == 0.5
  assert "rewards/sum" not in out["log_metrics"]
  both = reward_manager.AgenticSequenceRewardManager([length], Cfg())(PROMPTS, DONE, trajectory_rewards=[1.0, 0.0, 0.5])
  assert both["rewards"].tolist() == [2.0, 4.0, 3.5] and "rewards/length" in both["log_metrics"]


# ---- algorithm configuration ----------------------------------------------------------------------------
def test_algorithm_config_checks_names_once_and_has_no_room_for_typos(caplog):
  with caplog.at_level(logging.INFO):
    c = algorithm_config.AlgorithmConfig(algo_variant="gspo-token", advantage_estimator="gae", policy_loss_fn="ppo")
  assert "Initializing AlgorithmConfig" in caplog.text and "advantage_estimator: gae" in caplog.text
  d = algorithm_config.AlgorithmConfig()
  assert (d.algo_variant, d.advantage_estimator, d.policy_loss_fn, d.kl_clamp_value) == ("grpo", "grpo", "grpo", None)
  assert algorithm_config.AlgorithmConfig(kl_clamp_value=10.0).kl_clamp_value == 10.0
  for field, bad in [("algo_variant", "grpo-x"), ("advantage_estimator", ""), ("policy_loss_fn", "PPO")]:
    with pytest.raises(ValueError, match=field):
      algorithm_config.AlgorithmConfig(**{field: bad})
  with pytest.raises(TypeError):
    algorithm_config.AlgorithmConfig("grpo", "grpo", "grpo")
  with pytest.raises(AttributeError):
    d.new_attribute = 1
  d.algo_variant = "not checked after construction"
  assert d.algo_variant.startswith("not checked")


# ---- progress bar and TFLOPs ----------------------------------------------------------------------------
def test_progress_bar_shows_training_before_evaluation_and_rounds(caplog, monkeypatch):
  lg = ml.MetricsLogger()
  lg.log("actor", "loss", 0.91234, "eval", 0)
  lg.log("actor", "loss", 1.23456, "train", 0)
  lg.log("actor", "perplexity", 3.4366, "train", 0)
  monkeypatch.setattr(progress_bar, "_is_in_ipython", lambda: True)      # a disabled bar does not count steps
  pb = progress_bar.ProgressBar(lg, initial_steps=0, max_steps=4, description="t", metrics_prefix="actor")
  assert pb.metrics == {}
  pb.update_metrics(["loss"], ml.Mode.EVAL)
  with caplog.at_level(logging.WARNING):
    pb.update_metrics(["loss", "perplexity", "learning_rate", "missing"], "train", ndigits=2)
  assert list(pb.metrics.items()) == [("actor_train_loss", 1.23), ("actor_train_perplexity", 3.44), ("actor_eval_loss", 0.912)]
  assert "Metric missing not found for mode train" in caplog.text and "learning_rate" not in caplog.text
  pb.update(); pb.update(2)
  assert pb.tqdm_bar.n == 3
  pb.close(); pb.close()
  for tty, notebook, disabled in [(True, False, False), (False, True, False), (False, False, True)]:
    monkeypatch.setattr("sys.stderr.isatty", lambda tty=tty: tty, raising=False)
    monkeypatch.setattr(progress_bar, "_is_in_ipython", lambda notebook=notebook: notebook)
    bar = progress_bar.ProgressBar(lg, 0, 2, metrics_prefix="actor")
    assert bar.tqdm_bar.disable == disabled
    bar.close()


def test_tflops_estimates(caplog):
  assert smc.approximate_tflops_per_second(10**9, 4096, 2.0) == pytest.approx(6 * 4096 * 1e9 / 2.0 / 1e12)
  with caplog.at_level(logging.WARNING):
    assert smc.approximate_tflops_per_second(10**9, 4096, 0.0) == 0.0
    assert smc.approximate_tflops_per_second(0, 4096, 1.0) == 0.0
  assert caplog.text.count("TFLOPS cannot be approximated") == 2
  from tests.test_rl_grpo import toy_model
  from tunix_b200.models import flops
  m = toy_model()
  assert smc.measure_tflops_per_step(m, 1024, seq_len=128) == pytest.approx(
      flops.train_flops_per_token(m.config, 128) * 1024 / 1e12)

  class Bare:
    def parameters(self):
      import torch
      return [torch.zeros(10, 10)]
  assert smc.measure_tflops_per_step(Bare(), 1000) == pytest.approx(6 * 100 * 1000 / 1e12)
  assert smc.measure_tflops_per_step(object(), 1000) is None
