"""The remote-execution demos: registry-built agents and environments on the worker, a request served over gRPC,
and the epoch loop over a pool with out-of-order completion, a failing request and weight-version pushes."""
import asyncio
import pickle

import pytest

from tunix_b200.experimental.common import datatypes
from tunix_b200.experimental.rl.agentic import registry
from tunix_b200.experimental.worker import remote_execution
from tunix_b200.experimental.worker.examples import (agentic_remote_execution_demo as demo,
                                                     rl_loop_remote_execution_demo as loop_demo, sample_agent_and_env)


def test_the_sample_parts_register_themselves_and_the_client_stays_where_it_was_built():
  names = registry.auto_discover_modules(demo.EXAMPLES_PACKAGE)
  assert any(n.endswith("sample_agent_and_env") for n in names)
  assert registry.AGENT_REGISTRY.get("triage") is sample_agent_and_env.TriageAgent
  assert registry.ENV_REGISTRY.get("cluster") is sample_agent_and_env.ClusterTaskEnv
  env = sample_agent_and_env.ClusterTaskEnv(task={"node": "node-13"})
  with pytest.raises(TypeError, match="cannot be pickled"):
    pickle.dumps(env.client)
  obs, _ = env.reset()
  assert "node-13" in obs["observation"]
  agent = sample_agent_and_env.TriageAgent("sys")
  missed = env.step(agent.step(obs, difficulty="easy"))
  assert missed[1] == 0.0 and missed[2] is True                    # `uptime` calls the faulty node healthy
  env2 = sample_agent_and_env.ClusterTaskEnv(task={"node": "node-13"})
  env2.reset()
  found = env2.step(agent.step(obs, difficulty="hard"))
  assert found[1] == 1.0 and found[0].endswith("DEGRADED")
  env.close()
  with pytest.raises(RuntimeError, match="disconnected"):
    env.client.run("node-1", "uptime")


def test_one_request_is_served_by_a_worker_behind_grpc():
  response = asyncio.run(demo.demo())
  assert isinstance(response, datatypes.RolloutResponse) and response.status == "SUCCEEDED"
  assert response.request_id == "req-1" and response.env_reward == 1.0
  assert response.metadata["worker_id"] == "rollout-worker-1" and "ecc.errors" in response.metadata["action"]
  assert response.metadata["observation"].endswith("DEGRADED")


def test_the_worker_builds_agent_and_environment_per_request_and_names_unknown_types():
  async def go():
    w = demo.RegistryRolloutWorker("w0")
    assert w.state == datatypes.WorkerState.PENDING
    ok = await w.generate(datatypes.RolloutRequest(request_id="a", prompt="look at it", prompt_id="p",
                                                   metadata={"node": "node-2", "difficulty": "easy"}))
    assert w.state == datatypes.WorkerState.READY and ok.env_reward == 1.0 and w.served == 1
    assert w.sync_weights(4).metadata["policy_version"] == 4 and w.heartbeat().policy_version == 4
    with pytest.raises(KeyError, match="not registered"):
      await w.generate(datatypes.RolloutRequest(request_id="b", prompt="x", prompt_id="p", metadata={"env_type": "mars"}))
    assert w.info().roles == frozenset({"rollout"})
    w.stop()
    assert w.state == datatypes.WorkerState.STOPPED
  asyncio.run(go())


def test_the_epoch_loop_streams_results_from_every_worker_and_pushes_versions():
  report = asyncio.run(loop_demo.demo(workers=3, epochs=2, batch_size=6))
  assert [r["epoch"] for r in report] == [0, 1] and [r["policy_version"] for r in report] == [1, 2]
  for row in report:
    assert row["completed"] == 6 and row["failed"] == 0 and row["stale"] == 0 and len(row["workers"]) >= 2
    assert 0.0 <= row["avg_reward"] <= 1.0
  batches = loop_demo.synthetic_prompt_batches(2, 3, seed=1)
  assert batches == loop_demo.synthetic_prompt_batches(2, 3, seed=1) and len(batches) == 2 and len(batches[0]) == 3
  assert batches[1][2]["prompt_id"] == "prompt_b1_i2" and batches[0][0]["env_type"] == "cluster"


def test_a_failing_request_costs_only_itself():
  async def go():
    class Flaky(demo.RegistryRolloutWorker):
      async def generate(self, request):
        if request.request_id.endswith("_req_1"):
          raise RuntimeError("environment crashed")
        return await super().generate(request)
    servers = [remote_execution.InProcessRemoteExecutionServer(Flaky(f"w{i}", max_delay_s=0.02, seed=i)) for i in range(2)]
    handles = [remote_execution.InProcessActorHandle(s) for s in servers]
    return await loop_demo.run_rl_training_loop(handles, num_epochs=2, batch_size=4)
  report = asyncio.run(go())
  assert [(r["completed"], r["failed"]) for r in report] == [(3, 1), (3, 1)]
