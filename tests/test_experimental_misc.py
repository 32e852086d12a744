"""Trajectory schema and stores, agentic registry, process runtime, deployment."""

import argparse
import os
import sys
import textwrap
import threading

import numpy as np
import pytest
import yaml

from tunix_b200.experimental.trajectory import trajectory as T
from tunix_b200.experimental.trajectory import (
    FileTrajectoryStore, InMemoryTrajectoryStore, TrajectoryNotFoundError,
    TrajectoryReader, TrajectoryWriter)
from tunix_b200.experimental.rl.agentic import registry as R
from tunix_b200.experimental.distributed.runtime import main as rt_main
from tunix_b200.experimental.distributed.runtime import discovery
from tunix_b200.experimental.distributed.runtime.executor import (
    K8sExecutor, LocalExecutor)
from tunix_b200.experimental.distributed.runtime.executors import k8s_executor
from tunix_b200.experimental.distributed.deployment import yaml_generator


def _traj(tid="t0"):
  t = T.TunixTrajectory(agent=T.Agent(name="a", version="1"), trajectory_id=tid,
                        prompt_id="p", group_offset_id="0")
  t.add_step(T.Source.USER, "2+2?", env_tokens=[5, 6, 7])
  t.add_step(T.Source.AGENT, "4", assistant_tokens=[8, 9],
             logprobs=[-0.5, -0.25], policy_version=2,
             tool_calls=[T.ToolCall(tool_call_id="c1", function_name="calc",
                                    arguments={"e": "2+2"})],
             observation=T.Observation(results=[
                 T.ObservationResult(source_call_id="c1", content="4")]))
  t.add_step(T.Source.USER, "right", reward=1.0, done=True)
  return t


def test_trajectory_schema_rules():
  t = _traj()
  assert [s.step_id for s in t.steps] == [0, 1, 2]
  back = T.TunixTrajectory.from_json_dict(t.to_json_dict())
  assert isinstance(back.steps[1], T.TunixAgentStep)
  assert isinstance(back.steps[2], T.TunixEnvStep)
  toks, masks, lps = back.flat_tokens()
  np.testing.assert_array_equal(toks, [5, 6, 7, 8, 9])
  np.testing.assert_array_equal(masks, [0, 0, 0, 1, 1])
  np.testing.assert_allclose(lps, [0, 0, 0, -0.5, -0.25])
  assert back.sum_rewards() == 1.0
  assert back.get_metadata().prompt_id == "p"
  with pytest.raises(Exception, match="only allowed when source is 'agent'"):
    T.Step(step_id=1, source="user", model_name="m")
  with pytest.raises(Exception, match="only applicable when source is 'agent'"):
    T.TunixAgentStep(step_id=0, source="user")
  with pytest.raises(Exception, match="sequential from 1"):
    T.Trajectory(agent=T.Agent(name="a"),
                 steps=[T.Step(step_id=2, source="user")])
  with pytest.raises(Exception, match="unknown tool call"):
    T.Step(step_id=1, source="agent",
           tool_calls=[T.ToolCall(tool_call_id="a", function_name="f")],
           observation=T.Observation(results=[
               T.ObservationResult(source_call_id="zzz")]))
  with pytest.raises(Exception, match="duplicate ID"):
    T.Trajectory(agent=T.Agent(name="a"), subagent_trajectories=[
        T.Trajectory(agent=T.Agent(name="b"), trajectory_id="s"),
        T.Trajectory(agent=T.Agent(name="c"), trajectory_id="s")])
  with pytest.raises(Exception):
    T.Step(step_id=1, source="user", bogus=1)
  plain = T.Trajectory(agent=T.Agent(name="a"))
  plain.add_step(T.Source.SYSTEM, "sys")
  plain.add_step(T.Source.AGENT, "hi", model_name="m")
  assert plain.to_json_dict()["schema_version"] == "ATIF-v1.7"
  assert [s.step_id for s in plain.steps] == [1, 2]


@pytest.mark.parametrize("kind", ["memory", "file"])
def test_trajectory_stores(tmp_path, kind):
  if kind == "memory":
    st = InMemoryTrajectoryStore(trajectory_cls=T.TunixTrajectory)
  else:
    st = FileTrajectoryStore(str(tmp_path / "run"),
                             trajectory_cls=T.TunixTrajectory)
  assert isinstance(st, TrajectoryReader) and isinstance(st, TrajectoryWriter)
  assert st.get_trajectories_metadata() == []
  for tid in ("a", "b"):
    t = _traj(tid)
    for s in t.steps:
      st.add_step(s, t.get_metadata())
      s.message = "mutated after logging"      # the store took a snapshot
  meta = _traj("a").get_metadata()
  meta.total_reward = 3.5
  st.update_metadata(meta)
  st.flush()
  ids = sorted(m.trajectory_id for m in st.get_trajectories_metadata())
  assert ids == ["a", "b"]
  got = st.get_trajectories(["b", "a"])
  assert [g.trajectory_id for g in got] == ["b", "a"]
  assert got[0].steps[1].message == "4"
  assert got[1].total_reward == 3.5
  np.testing.assert_array_equal(got[0].steps[1].assistant_tokens, [8, 9])
  with pytest.raises(TrajectoryNotFoundError):
    st.get_trajectories(["nope"])
  with pytest.raises(ValueError):
    st.update_metadata(T.TunixTrajectoryMetadata(agent=T.Agent(name="a"),
                                                 trajectory_id="../x"))
  if kind == "file":
    assert os.path.isfile(st.get_step_path("a", 2))
    st.close()


def test_file_store_survives_io_errors(tmp_path):
  root = tmp_path / "blocked"
  root.write_text("a file where the directory should be")
  st = FileTrajectoryStore(str(root), trajectory_cls=T.TunixTrajectory)
  t = _traj("x")
  st.add_step(t.steps[0], t.get_metadata())
  st.flush()                       # the failure is logged, not raised
  assert st._writer.errors == 1
  st.close()


def test_registry_and_discovery(tmp_path):
  reg = R.Registry("Things")

  @reg.register("one")
  class A:
    pass

  @reg.register()
  class B:
    pass

  @reg.register
  class C:
    pass

  assert reg.keys() == ["B", "C", "one"] and reg.get("one") is A
  assert "B" in reg and not reg.contains("zzz")
  with pytest.raises(KeyError, match="not registered"):
    reg.get("zzz")
  with pytest.raises(ValueError, match="already registered"):
    reg.register("one")(B)

  plug = tmp_path / "plugins"
  plug.mkdir()
  (plug / "mine.py").write_text(textwrap.dedent("""
      from tunix_b200.experimental.rl.agentic.registry import register_agent as ra
      @ra("discovered_agent")
      class Mine:
        pass
  """))
  (plug / "other.py").write_text("raise RuntimeError('must not be imported')\n")
  (plug / "broken.py").write_text("def (:\n")
  assert R.has_registry_decorator(str(plug / "mine.py"))
  assert not R.has_registry_decorator(str(plug / "other.py"))
  assert not R.has_registry_decorator(str(plug / "broken.py"))
  names = R.auto_discover_modules(str(plug))
  assert len(names) == 1 and "discovered_agent" in R.AGENT_REGISTRY


_heard = []
_done = threading.Event()


def door_main(ctx, argv):
  ctx.ipc.discovery.on_register(
      lambda host, port, meta: (_heard.append((host, port, meta)), _done.set()))
  assert _done.wait(20)


def knocker_main(ctx, argv):
  p = argparse.ArgumentParser()
  p.add_argument("--say")
  ctx.ipc.discovery.register(p.parse_args(argv).say.encode())


def test_runtime_door_and_knocker():
  import socket
  with socket.socket() as s:
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
  assert rt_main.split_process_argv(["--process", "a", "--process", "b", "c"]) \
      == [["a"], ["b", "c"]]
  me = __name__
  sys.modules.setdefault(me, sys.modules[__name__])
  rt_main.main([
      "prog", "--process",
      f"--process_main={me}.door_main", "--discovery_id=door",
      f"--discovery_port={port}",
      "--process", f"--process_main={me}.knocker_main",
      "--discovery_id=knocker", f"--discovery_addrs=door:{port}",
      "--say=open the door"])
  assert _heard == [("knocker", 0, b"open the door")]
  with pytest.raises(ValueError, match="Invalid --process_main"):
    rt_main.prepare_process(["--process_main=os.nothing_here"])
  assert discovery.parse_addrs("a:1, b:22") == [("a", 1), ("b", 22)]
  with pytest.raises(ValueError):
    discovery.parse_addrs("nohost")
  assert LocalExecutor and K8sExecutor
  assert k8s_executor.pod_dns_name("js", "rollout") == "js-rollout-0-0.js"


def test_deployment_yaml(tmp_path):
  d = os.path.dirname(yaml_generator.__file__)
  out = tmp_path / "o.yaml"
  yaml_generator.main([
      os.path.join(d, "yamls", "jobset.gpu.yaml"), "--gpu_slice", "b200:2x8",
      "--jobset_name", "js", "--worker_startup_command", "python bench.py",
      "-o", str(out)])
  doc = yaml.safe_load(out.read_text())
  job = doc["spec"]["replicatedJobs"][0]["template"]["spec"]
  assert job["completions"] == 2 and job["parallelism"] == 2
  c = job["template"]["spec"]["containers"][0]
  assert c["resources"]["limits"]["nvidia.com/gpu"] == 8
  assert "--nnodes=2 --nproc-per-node=8" in c["command"][-1]
  assert "--master-addr=js-proc-0-0.js" in c["command"][-1]
  cpu = yaml_generator.render(
      open(os.path.join(d, "yamls", "jobset.cpu.yaml")).read(),
      yaml_generator.build_parser().parse_args(
          ["x", "--cpu_machine", "n2-standard-64"]), environ={"USER": "u"})
  assert yaml.safe_load(cpu)["metadata"]["name"] == "u-cpu"
  with pytest.raises(ValueError):
    yaml_generator.parse_gpu_slice("tpu7x:4x4")
  with pytest.raises(ValueError):
    yaml_generator.parse_gpu_slice("b200:2x4")


def test_mock_parts_drive_collect_train_sync():
  """`experimental/common/test_utils.py`: the stand-ins behave like the parts they replace."""
  import asyncio
  import threading
  from tunix_b200.experimental.common import test_utils as tu
  from tunix_b200.experimental.rollout import sampler as sampler_lib
  tok = tu.MockTokenizer()
  assert tok.decode(tok.encode("héllo", add_special_tokens=True)) == "héllo"
  assert tok.dedup_bos_ids([1, 1, 1, 7]) == [1, 7] and tok.dedup_bos_ids([1, 7]) == [1, 7]
  parser = tu.MockChatParser()
  assert parser.parse([{"role": "user", "content": "hi"}], add_generation_prompt=True) == "<user>hi</user><assistant>"
  # the pool blocks when empty and refuses a double release
  pool = tu.MockEnvironmentPool(1)
  env = pool.acquire_env()
  with pytest.raises(TimeoutError):
    pool.acquire_env(timeout=0.05)
  threading.Timer(0.05, pool.release_env, args=(env,)).start()
  assert pool.acquire_env(timeout=2.0) is env
  pool.release_env(env)
  with pytest.raises(ValueError):
    pool.release_env(env)
  # an episode: keywords rewarded turn by turn, done after `turns`
  e = tu.MockEnvironment(delay_seconds=0.0, turns=2)
  obs, _ = e.reset()
  assert "alpha" in obs["question"]
  obs, r, done, info = e.step("alpha please")
  assert r == 1.0 and not done and "beta" in obs["question"]
  _, r, done, _ = e.step("wrong")
  assert r == 0.0 and done
  # the sampler follows the protocol, truncates at max_tokens and answers "cancelled" while paused
  s = tu.MockSampler()
  assert isinstance(s, sampler_lib.Sampler)

  async def sampling():
    full = (await s.sample([sampler_lib.SamplingRequest(prompt="x")]))[0]
    short = (await s.sample([sampler_lib.SamplingRequest(
        prompt="x", sampling_params=sampler_lib.SamplingParams(max_tokens=3, return_logprobs=True))]))[0]
    await s.pause()
    cancelled = (await s.sample([sampler_lib.SamplingRequest(prompt="x")]))[0]
    await s.resume()
    return full, short, cancelled
  full, short, cancelled = asyncio.run(sampling())
  assert full.finish_reason == "stop" and short.finish_reason == "length" and len(short.token_ids) == 3
  assert short.logprobs.shape == (3,) and cancelled.finish_reason == "cancelled"
  # collect -> train -> sync, twice: rewards are earned, versions advance, the sampler saw every phase
  orch = tu.MockGlobalOrchestrator(num_envs=2)
  with pytest.raises(RuntimeError):
    asyncio.run(orch.collect_rollout_batch(1))
  orch.start_workers()
  for round_ in (1, 2):
    batch = asyncio.run(orch.collect_rollout_batch(4))
    assert len(batch) == 4 and all(ep.steps == 2 and ep.reward == 2.0 for ep in batch)
    assert all(ep.policy_version == round_ - 1 for ep in batch)
    assert asyncio.run(orch.run_training_step(batch)) == round_
    assert orch.synchronize_weights(["rollout:0"]) == round_
  assert orch.sampler.policy_version == 2 and orch.trainer.mean_reward == 2.0
  assert orch.sampler.phases == ["pre", "transfer", "post"] * 2 and orch.pool.available == 2
  orch.stop_workers()
