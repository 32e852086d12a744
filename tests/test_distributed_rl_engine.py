"""`DistributedRLEngine` and `GroupExpansion` against in-process worker handles: group expansion and request ids,
prefix routing, polling and conversion of responses, call-and-wait generation, role lookup for training / scoring,
and weight sync through a coordinator."""
import asyncio

import numpy as np
import pytest

from tunix_b200.experimental.common import datatypes
from tunix_b200.experimental.orchestrator import distributed_rl_engine as dre, rl_engine_interface as iface
from tunix_b200.experimental.worker import remote_execution as rx


class RolloutWorker:
  """Answers every request with a two-token completion; remembers what it was asked."""

  def __init__(self, name):
    self.name, self.requests, self.prompts, self.kwargs = name, [], [], []

  def _answer(self, r):
    seg = datatypes.TokenSegment(source="assistant", tokens=np.array([7, 8]), loss_mask=np.array([1, 1]),
                                 logps=np.array([-0.5, -0.25]))
    return datatypes.RolloutResponse(request_id=r.request_id, prompt_id=r.prompt_id, status="COMPLETED",
                                     prompt_tokens=np.array([1, 2, 3]), segments=[seg], env_reward=1.5,
                                     policy_version=r.target_policy_version,
                                     metadata={**r.metadata, "worker": self.name})

  def generate(self, requests=None, prompts=None, **kwargs):
    self.kwargs.append(kwargs)
    out = []
    for r in requests or []:
      self.requests.append(r)
      out.append(self._answer(r))
    for p in prompts or []:
      self.prompts.append(p)
      out.append(self._answer(datatypes.RolloutRequest(request_id=f"adhoc-{p}", prompt=p, prompt_id=str(p))))
    return out


class Trainer:
  def __init__(self):
    self.calls = []

  def train_step(self, payload, accumulate_gradients, apply_optimizer, **kw):
    self.calls.append((payload, accumulate_gradients, apply_optimizer, kw))
    return {"loss": 1.0, "applied": apply_optimizer}


class Scorer:
  def score(self, items, **kw):
    return [float(len(i)) for i in items]

  def per_token_logps(self, items, **kw):
    return datatypes.LogprobsResponse(per_token_logps=np.full((len(items), 2), -1.0, np.float32))


def handle(obj):
  return rx.InProcessActorHandle(rx.InProcessRemoteExecutionServer(obj))


def engine(n_rollout=2, coordinator=None, inference=True):
  workers = [RolloutWorker(f"r{i}") for i in range(n_rollout)]
  trainer = Trainer()
  eng = dre.DistributedRLEngine([handle(w) for w in workers], {datatypes.Role.ACTOR: handle(trainer)},
                                {datatypes.Role.REFERENCE: handle(Scorer())} if inference else None, coordinator)
  return eng, workers, trainer


# ---- group expansion --------------------------------------------------------------------------------
def test_expansion_builds_one_group_per_prompt_with_stable_ids_and_routing_keys():
  plan = iface.GroupExpansion(group_size=3, policy_version=4, generation={"temperature": 0.7},
                              metadata={"run": "x"})
  items = [{"prompt_id": "p0", "prompt": "hello", "generation_kwargs": {"temperature": 0.1, "top_k": 5},
            "metadata": {"env_config": {"seed": 9}}, "max_turns": 2},
           type("Item", (), {"prompt_id": 7, "prompt": "object", "group_id": "g7"})()]
  reqs = list(plan.requests(items))
  assert [r.request_id for r in reqs[:3]] == ["req_p0_0_v4", "req_p0_1_v4", "req_p0_2_v4"]
  assert iface.request_id("p0", 2, 4) == reqs[2].request_id
  first = reqs[0]
  assert first.prompt == "hello" and first.group_offset_id == "0" and first.target_policy_version == 4
  assert first.generation_kwargs == {"temperature": 0.1, "top_k": 5} and first.max_turns == 2     # the item's own win
  assert first.metadata["run"] == "x" and first.metadata["group_id"] == "p0" and first.metadata["prefix_hash"] == "p0"
  assert [r.metadata["pair_index"] for r in reqs[:3]] == [0, 1, 2]
  assert reqs[1].metadata["env_config"] == {"group_id": "p0", "seed": 9, "pair_index": 1, "policy_version": 4}
  assert reqs[3].prompt_id == "7" and reqs[3].metadata["group_id"] == "g7" and reqs[3].max_turns == 10
  assert reqs[0].traj_id == "traj_p0_0"
  ready = datatypes.RolloutRequest(request_id="mine", prompt="x", prompt_id="px")
  assert list(plan.requests([ready])) == [ready]                                             # passes through
  with pytest.raises(ValueError, match="index 1 lacks 'prompt_id'"):
    list(plan.requests([{"prompt_id": "a", "prompt": "1"}, {"prompt": "2"}]))


# ---- fire and collect ---------------------------------------------------------------------------------
def test_samples_of_a_prompt_land_on_one_worker_and_come_back_as_trajectory_items():
  eng, workers, _ = engine()

  async def scenario():
    ids = await eng.dispatch_rollouts([{"prompt_id": f"p{i}", "prompt": f"q{i}"} for i in range(6)], group_size=2,
                                      policy_version=3, generation_args=datatypes.GenerationArgs(temperature=0.5),
                                      route_metadata={"tenant": "t"})
    items = []
    for _ in range(50):
      items += await eng.poll_rollouts(timeout_s=0.05)
      if len(items) == 12:
        break
    return ids, items
  ids, items = asyncio.run(scenario())
  assert len(ids) == 12 and ids[0] == "req_p0_0_v3"
  by_prompt = {}
  for w in workers:
    for r in w.requests:
      by_prompt.setdefault(r.prompt_id, set()).add(w.name)
      assert r.generation_kwargs == {"temperature": 0.5} and r.metadata["tenant"] == "t"
  assert all(len(names) == 1 for names in by_prompt.values()) and len(by_prompt) == 6      # a group never splits
  assert sum(len(w.requests) for w in workers) == 12 and all(w.requests for w in workers)   # and both workers got work
  assert len(items) == 12 and all(isinstance(it, datatypes.TrajectoryItem) for it in items)
  one = next(it for it in items if it.group_id == "p0" and it.pair_index == 1)
  assert one.prompt_tokens.tolist() == [1, 2, 3] and one.completion_tokens.tolist() == [7, 8]
  assert one.action_mask.tolist() == [1, 1] and one.policy_version == 3 and one.traj.reward == 1.5
  assert one.metadata["old_logps"].tolist() == [-0.5, -0.25] and one.metadata["status"] == "COMPLETED"


def test_polling_survives_a_broken_worker_and_an_engine_without_workers():
  eng, workers, _ = engine()

  async def boom(timeout_s=0.0, max_items=64):
    raise ConnectionError("worker 1 is down")
  eng._rollout_workers[1].poll_responses = boom

  async def scenario():
    await eng.dispatch_rollouts([{"prompt_id": "solo", "prompt": "q"}], group_size=1)
    got = []
    for _ in range(20):
      got += await eng.poll_rollouts(timeout_s=0.02)
    return got
  got = asyncio.run(scenario())
  assert len(got) <= 1                                     # whatever the healthy worker had; no exception
  empty = dre.DistributedRLEngine([], {})
  assert asyncio.run(empty.poll_rollouts(timeout_s=0.0)) == []
  with pytest.raises(ValueError, match="no registered rollout workers"):
    asyncio.run(empty.generate(["x"]))


def test_error_responses_keep_their_message():
  failed = datatypes.RolloutResponse(request_id="r", prompt_id="p", status="FAILED",
                                     error=datatypes.ErrorInfo(error_type="Timeout", message="env timed out"))
  item = dre._response_to_trajectory_item(failed)
  assert item.metadata["error"] == "env timed out" and item.metadata["status"] == "FAILED" and item.group_id == "p"
  assert len(item.completion_tokens) == 0
  same = datatypes.TrajectoryItem(pair_index=0, group_id="g", start_step=0, traj=datatypes.Trajectory(reward=0.0))
  assert dre._response_to_trajectory_item(same) is same


# ---- call and wait ------------------------------------------------------------------------------------
def test_generate_takes_explicit_generation_args_only():
  eng, workers, _ = engine()
  out = asyncio.run(eng.generate(["a", "b"], generation_args=datatypes.GenerationArgs(max_generation_steps=4, top_p=0.9),
                                 route_metadata={"prompt_id": "same"}))
  assert len(out) == 2 and sum(len(w.prompts) for w in workers) == 2
  used = [w for w in workers if w.prompts]
  assert len(used) == 1 and used[0].kwargs == [{"max_generation_steps": 4, "top_p": 0.9}]     # one routing key, one call
  with pytest.raises(TypeError, match="Use generation_args=GenerationArgs"):
    asyncio.run(eng.generate(["a"], temperature=0.3))
  reqs = [datatypes.RolloutRequest(request_id=f"x{i}", prompt="p", prompt_id=f"p{i}") for i in range(4)]
  out = asyncio.run(eng.generate(reqs))
  assert sorted(it.metadata["worker"] for it in out).count("r0") + sorted(it.metadata["worker"] for it in out).count("r1") == 4


# ---- roles ----------------------------------------------------------------------------------------------
def test_training_and_scoring_go_to_the_role_handles():
  eng, _, trainer = engine()
  res = asyncio.run(eng.train_step({"tokens": 1}, accumulate_gradients=True, apply_optimizer=False, extra=5))
  assert res == {"loss": 1.0, "applied": False} and trainer.calls == [({"tokens": 1}, True, False, {"extra": 5})]
  assert asyncio.run(eng.train_step("p", role="actor"))["applied"]              # role by value or by enum
  with pytest.raises(ValueError, match="no trainer worker registered for role"):
    asyncio.run(eng.train_step("p", role=datatypes.Role.CRITIC))
  assert asyncio.run(eng.score(datatypes.Role.REFERENCE, ["ab", "c"])) == [2.0, 1.0]
  lp = asyncio.run(eng.per_token_logps(datatypes.Role.REFERENCE, items=["x", "y", "z"]))
  assert lp.shape == (3, 2)                                                      # the response object is unwrapped
  no_inference, _, _ = engine(inference=False)
  with pytest.raises(ValueError, match="no inference worker registered"):
    asyncio.run(no_inference.score(datatypes.Role.REWARD, []))


def test_weight_sync_asks_the_coordinator_and_counts_versions():
  class Coordinator:
    def __init__(self): self.versions = []
    async def sync(self, version):
      self.versions.append(version)
  co = Coordinator()
  eng, _, _ = engine(coordinator=co)
  assert asyncio.run(eng.sync_weights()) == 1 and asyncio.run(eng.sync_weights()) == 2
  assert co.versions == [1, 2] and eng.policy_version == 2

  class Failing:
    async def sync(self, version):
      raise RuntimeError("round aborted")
  eng2, _, _ = engine(coordinator=Failing())
  with pytest.raises(RuntimeError, match="round aborted"):
    asyncio.run(eng2.sync_weights())
  assert eng2.policy_version == 0                                                # a failed round publishes nothing
  standalone, _, _ = engine()
  assert asyncio.run(standalone.sync_weights()) == 1                             # colocated weights: versions only


def test_the_managed_run_with_simulated_workers_routes_groups_and_trains(capsys):
  from tunix_b200.experimental.common import datatypes as dt
  from tunix_b200.experimental.orchestrator import simple_orchestrator_nb as nb
  out = nb.main(num_steps=2, group_size=2)
  assert [r.step for r in out["history"]] == [0, 1] and all(r.num_rollouts == 4 for r in out["history"])
  assert out["optimizer_steps"] == 2 and out["trainer_batches"] == 4
  # both samples of a prompt were served by the same worker
  owner = {}
  for worker, served in out["served"].items():
    for request_id in served:
      prompt = request_id.split("_")[1]
      assert owner.setdefault(prompt, worker) == worker
  assert sum(len(s) for s in out["served"].values()) == 8
  assert set(out["states"].values()) == {dt.WorkerState.STOPPED}
  assert "reward mean" in capsys.readouterr().out
  again = nb.main(num_steps=2, group_size=2)                  # deterministic
  assert [r.reward_mean for r in again["history"]] == [r.reward_mean for r in out["history"]]
