"""More of the trajectory collection engine: result modes, synchronous and asynchronous model calls, list-valued
log-probs, concurrent collection, the overlong filter with and without a final reward, timing records, span tags,
and misuse."""
import asyncio
import time

import numpy as np
import pytest

from tunix_b200.rl.agentic.agents import agent_types, model_agent
from tunix_b200.rl.agentic.environments import base_environment
from tunix_b200.rl.agentic.parser.chat_template_parser import parser as ctp
from tunix_b200.rl.agentic.trajectory.trajectory_collect_engine import TrajectoryCollectEngine
from tests.test_agentic import CharTok, out

Status = agent_types.TrajectoryStatus


class CountingEnv(base_environment.BaseTaskEnv):
  """A multi-turn task: the episode ends when the answer is "done" or after `max_steps`."""

  def __init__(self, task, *, latency=0.0, **kw):
    super().__init__(task, **kw)
    self.latency, self.closed = latency, 0

  def _initial_observation(self):
    return {"question": self.task["question"]}

  def _step_impl(self, action):
    if self.latency:
      time.sleep(self.latency)
    if str(action).strip() == "done":
      return self.final(action)
    return self.turn({"question": f"again ({self.step_count})"}, response=action, reward=0.25)

  def close(self):
    self.closed += 1


def engine(replies, env=None, **kw):
  replies = iter(replies)
  env = env or CountingEnv({"question": "say done"}, reward_fn=lambda task, action: 1.0, max_steps=4, pair_index=1, group_id="g")
  tok = CharTok()
  kw.setdefault("tokenizer", tok)
  kw.setdefault("chat_parser", ctp.QwenChatTemplateParser(tok))
  kw.setdefault("model_call", lambda msgs, env, **k: out(next(replies)))
  return TrajectoryCollectEngine(model_agent.ModelAgent("sys"), env, **kw), env


def test_result_modes_describe_the_same_episode():
  results = {}
  for mode in ("Trajectory", "Conversation", "Steps", "Token"):
    eng, env = engine(["hm", "done"], gamma=0.5)
    results[mode] = asyncio.run(eng.collect(mode))
    assert env.closed == 1
  traj = results["Trajectory"]
  assert traj.status == Status.SUCCEEDED and len(traj.steps) == 2 and traj.reward == pytest.approx(1.25)
  assert [s.mc_return for s in traj.steps] == pytest.approx([0.25 + 0.5 * 1.0, 1.0])
  assert traj.env_time["step_latency"] and len(traj.env_time["step_latency"]) == 2 and "reward_latency" in traj.reward_time
  convo = results["Conversation"]
  assert [m["role"] for m in convo] == ["system", "user", "assistant", "user", "assistant"]
  steps = results["Steps"]
  assert [s["assistant_text"] for s in steps] == ["hm", "done"] and [s["done"] for s in steps] == [False, True]
  assert len(steps[0]["env_tokens"]) > 0 and len(steps[1]["env_tokens"]) == 0        # nothing follows the last turn
  token = results["Token"]
  assert token["status"] == "SUCCEEDED" and token["trajectory_reward"] == pytest.approx(1.25) and token["group_id"] == "g"
  n = len(token["conversation_tokens"])
  assert len(token["conversation_masks"]) == n == len(token["old_logprobs"])
  trained = token["conversation_masks"].astype(bool)
  assert trained.sum() == len("hm") + len("done")                                   # only sampled tokens are trained on
  assert np.all(token["old_logprobs"][trained] == -0.5) and np.all(token["old_logprobs"][~trained] == 0.0)
  with pytest.raises(ValueError, match="Unsupported mode"):
    asyncio.run(engine(["done"])[0].collect("Video"))


def test_model_calls_may_be_coroutines_and_logprobs_plain_lists():
  seen = []

  async def acall(messages, env, **kw):
    seen.append(kw.get("max_generation_steps"))
    await asyncio.sleep(0.001)
    reply = out("done")
    reply.logprobs = [[-1.0, -2.0, -3.0, -4.0]]                                      # a list, not an array
    return reply
  eng, _ = engine([], model_call=acall, max_response_length=100, model_call_kwargs={"temperature": 0.3})
  token = asyncio.run(eng.collect("Token"))
  assert seen == [100] and token["old_logprobs"][:4].tolist() == [-1.0, -2.0, -3.0, -4.0]

  def failing(messages, env, **kw):
    raise ConnectionError("sampler is down")
  eng, env = engine([], model_call=failing)
  with pytest.raises(ConnectionError, match="sampler is down"):
    asyncio.run(eng.collect("Trajectory"))


def test_episodes_collected_together_finish_in_their_own_time():
  def pair(latency):
    env = CountingEnv({"question": "q"}, reward_fn=lambda task, action: 1.0, max_steps=2, latency=latency)
    return model_agent.ModelAgent("s"), env
  pairs = [pair(0.15), pair(0.0), pair(0.05)]

  async def run():
    order = []
    async for index, traj in TrajectoryCollectEngine.collect_multiple(pairs, model_call=lambda m, e, **k: out("done"),
                                                                      mode="Trajectory"):
      order.append((index, traj.status))
    return order
  t0 = time.perf_counter()
  order = asyncio.run(run())
  assert time.perf_counter() - t0 < 0.15 + 0.05 + 0.1                               # concurrent, not one after another
  assert [i for i, _ in order] == [1, 2, 0] and all(s == Status.SUCCEEDED for _, s in order)


def _limited(overlong_filter, final_reward=5.0, **kw):
  """The engine's own turn limit (2) is below the environment's (5): the episode is clipped, not finished."""
  env = CountingEnv({"question": "q"}, reward_fn=lambda task, action: 1.0, max_steps=5, pair_index=0)
  env.final_reward_fn = lambda: final_reward
  eng, _ = engine(["hm", "hm", "hm"], env=env, overlong_filter=overlong_filter, **kw)
  eng.max_steps = 2
  return asyncio.run(eng.collect("Token")), eng


def test_overlong_filter_masks_the_episode_and_skips_the_final_reward():
  token, eng = _limited(True)
  assert token["status"] == "MAX_STEPS_REACHED" and token["conversation_masks"].sum() == 0
  assert token["trajectory_reward"] == pytest.approx(0.25 * 2)                      # step rewards only
  assert len(token["conversation_tokens"]) == len(token["conversation_masks"]) > 0   # tokens kept, just not trained on
  kept, _ = _limited(False)
  assert kept["status"] == "MAX_STEPS_REACHED" and kept["conversation_masks"].sum() > 0
  assert kept["trajectory_reward"] == pytest.approx(0.25 * 2 + 5.0)                 # the final reward counts
  # the filter only looks at clipped episodes
  env = CountingEnv({"question": "q"}, reward_fn=lambda task, action: 1.0, max_steps=3, pair_index=0)
  env.final_reward_fn = lambda: 5.0
  eng, _ = engine(["done"], env=env, overlong_filter=True)
  fine = asyncio.run(eng.collect("Token"))
  assert fine["status"] == "SUCCEEDED" and fine["conversation_masks"].sum() == 4 and fine["trajectory_reward"] == 6.0
  custom, _ = _limited(True, filter_statuses={Status.TIMEOUT})
  assert custom["status"] == "MAX_STEPS_REACHED" and custom["conversation_masks"].sum() > 0   # not in the custom set


def test_whole_episode_timeout_and_latency_records():
  env = CountingEnv({"question": "q"}, reward_fn=lambda task, action: 1.0, max_steps=5, latency=0.06)
  eng, _ = engine(["hm"] * 5, env=env, timeout=0.1)
  traj = asyncio.run(eng.collect("Trajectory"))
  assert traj.status in (Status.TIMEOUT, Status.ENV_TIMEOUT) and len(traj.steps) <= 3 and traj.steps[-1].done
  assert all(dt >= 0.05 for dt in traj.env_time["step_latency"]) and traj.env_time["reset_latency"] >= 0.0
  assert env.closed == 1


def test_span_tags_come_from_the_environment():
  class Recorder:
    def __init__(self): self.spans = []
    def span(self, name, tags=None):
      self.spans.append((name, dict(tags or {})))
      import contextlib
      return contextlib.nullcontext()
  rec = Recorder()
  env = CountingEnv({"question": "q", "policy_version": 9}, reward_fn=lambda task, action: 1.0, max_steps=2, pair_index=3,
                    group_id="grp")
  eng, _ = engine(["done"], env=env, perf_v2=rec)
  asyncio.run(eng.collect("Trajectory"))
  assert rec.spans == [("environment", {"group_id": "grp", "pair_index": 3, "step": 9})]
  bare = CountingEnv({"question": "q"}, reward_fn=lambda task, action: 1.0, max_steps=2)
  assert engine(["done"], env=bare)[0]._perf_tags() == {}


def test_length_limits_need_a_tokenizer(caplog):
  with caplog.at_level("WARNING"):
    eng, _ = engine(["done"], tokenizer=None, chat_parser=None, max_response_length=10)
  assert "response length limits will not be enforced" in caplog.text
  token = asyncio.run(eng.collect("Token"))
  assert token["status"] == "SUCCEEDED" and len(token["conversation_tokens"]) == 0  # nothing is tokenised without one
