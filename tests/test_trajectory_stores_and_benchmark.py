"""Both trajectory stores against the conformance suite, the recovery benchmark (workload checks, generator, staged
run, a store that loses data, the command line), and the runtime's process contexts."""
import json
import os
import types

import pytest

from tunix_b200.experimental.distributed.runtime import context as rt_context
from tunix_b200.experimental.distributed.runtime.contexts import k8s_context, local_context
from tunix_b200.experimental.distributed.runtime.executors import k8s_executor, local_executor
from tunix_b200.experimental.trajectory import file_store, in_memory_store, store, store_testing
from tunix_b200.experimental.trajectory import trajectory as T
from tunix_b200.experimental.trajectory.benchmarks import benchmark_lib, data_generator, run_benchmark


class TestInMemoryStore(store_testing.StoreConformance):
  def make_store(self, tmp_path):
    return in_memory_store.InMemoryTrajectoryStore()


class TestFileStore(store_testing.StoreConformance):
  def make_store(self, tmp_path):
    return file_store.FileTrajectoryStore(str(tmp_path / "root"))

  def test_a_directory_without_metadata_is_its_own_error(self, rw, tmp_path):
    reader, _ = rw
    os.makedirs(tmp_path / "root" / "half_written")
    with pytest.raises(store.TrajectoryMetadataNotFoundError) as e:
      reader.get_trajectories(["half_written"])
    assert e.value.trajectory_id == "half_written"
    assert reader.get_trajectories_metadata() == []


class TestSeparateReaderAndWriter(store_testing.StoreConformance):
  """Two objects over one directory: what a trainer (writer) and a recovery tool (reader) are."""

  def make_store(self, tmp_path):
    root = str(tmp_path / "shared")
    return file_store.FileTrajectoryStore(root), file_store.FileTrajectoryStore(root)


# ---- benchmark ----------------------------------------------------------------------------------------
def test_workloads_are_checked():
  w = data_generator.WorkloadConfig(cumulative_trajectory_checkpoints=[2, 5], steps_per_trajectory=3, step_payload_chars=40)
  assert w.total_trajectories == 5
  for bad in ([], [0, 5], [5, 5], [5, 2], [1.5]):
    with pytest.raises(ValueError):
      data_generator.WorkloadConfig(cumulative_trajectory_checkpoints=bad)
  with pytest.raises(ValueError, match="steps_per_trajectory"):
    data_generator.WorkloadConfig(steps_per_trajectory=0)
  with pytest.raises(ValueError, match="step_payload_chars"):
    data_generator.WorkloadConfig(step_payload_chars=0)


def test_the_generator_is_lazy_numbered_from_one_and_tags_every_payload():
  w = data_generator.WorkloadConfig(cumulative_trajectory_checkpoints=[10**9], steps_per_trajectory=3, step_payload_chars=40)
  it = data_generator.generate_trajectories(w)              # a billion trajectories: only lazily possible
  meta, steps = next(it)
  assert meta.trajectory_id == "traj_000001" == data_generator.trajectory_id_of(1) and meta.agent.name == "benchmark_agent"
  assert [s.step_id for s in steps] == [1, 2, 3] and all(len(s.message) == 40 for s in steps)
  assert steps[1].message.startswith("[1:2]") and steps[1].message == data_generator.expected_message(w, 1, 2)
  assert next(it)[0].trajectory_id == "traj_000002"
  late = next(data_generator.generate_trajectories(w, first=77))
  assert late[0].trajectory_id == "traj_000077" and late[1][0].message.startswith("[77:1]")


def test_the_staged_run_reports_every_stage_and_verifies_content(tmp_path):
  w = data_generator.WorkloadConfig(cumulative_trajectory_checkpoints=[3, 8], steps_per_trajectory=4, step_payload_chars=64)
  lines = []
  st = file_store.FileTrajectoryStore(str(tmp_path / "bench"))
  report = benchmark_lib.run_recovery_benchmark(st, st, w, progress=lines.append)
  st.close()
  assert report.passed and report.reader_type == "FileTrajectoryStore" and report.workload is w
  assert [(c.checkpoint_write_count, c.total_trajectories) for c in report.checkpoints] == [(3, 3), (5, 8)]
  for c in report.checkpoints:
    assert c.write_qps > 0 and c.write_mb_per_sec > 0 and c.write_duration_sec > 0
    assert c.metadata_scan_latency_ms >= 0 and c.trajectory_load_latency_ms > 0 and c.validation_error is None
  assert any("[2/2]" in l and "ok" in l for l in lines)
  table = run_benchmark.format_report(report)
  assert "steps/s" in table and table.count("True") == 2
  assert len(os.listdir(tmp_path / "bench")) == 8


def test_a_store_that_loses_or_mixes_data_fails_the_stage_it_happened_in():
  class Forgetful(in_memory_store.InMemoryTrajectoryStore):
    def add_step(self, step, metadata):
      if metadata.trajectory_id != "traj_000004":
        super().add_step(step, metadata)
  w = data_generator.WorkloadConfig(cumulative_trajectory_checkpoints=[3, 5], steps_per_trajectory=2, step_payload_chars=16)
  st = Forgetful()
  first, second = benchmark_lib.run_recovery_benchmark(st, st, w, progress=None).checkpoints
  assert first.validation_passed and not second.validation_passed
  assert "traj_000004" in second.validation_error

  class Shuffling(in_memory_store.InMemoryTrajectoryStore):
    def get_trajectories(self, ids):
      out = super().get_trajectories(ids)
      out[0].steps[0].message = "someone else's payload"
      return out
  st = Shuffling()
  (only, _) = benchmark_lib.run_recovery_benchmark(st, st, w, progress=None).checkpoints
  assert not only.validation_passed and "different payload" in only.validation_error

  class Undercounting(in_memory_store.InMemoryTrajectoryStore):
    def get_trajectories_metadata(self):
      return super().get_trajectories_metadata()[1:]
  st = Undercounting()
  assert "metadata entries" in benchmark_lib.run_recovery_benchmark(st, st, w, progress=None).checkpoints[0].validation_error


def test_the_timer_is_reusable():
  t = benchmark_lib.Timer()
  with t:
    pass
  first = t.duration_sec
  assert first >= 0 and t.duration_ms == pytest.approx(first * 1e3)
  with t:
    sum(range(20000))
  assert t.duration_sec > 0


def test_the_command_line_runs_both_stores(tmp_path, capsys):
  cfg = run_benchmark.parse_args(["--store", "file", "--root_dir", str(tmp_path / "cli"), "--checkpoints", "2,4",
                                  "--steps", "2", "--payload_chars", "32", "--json"])
  assert isinstance(cfg.store, run_benchmark.FileTrajectoryStoreConfig) and cfg.workload.total_trajectories == 4
  report = run_benchmark.main(cfg)
  out = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
  assert report.passed and out["writer"] == "FileTrajectoryStore" and len(out["checkpoints"]) == 2
  assert out["workload"]["steps_per_trajectory"] == 2 and os.path.isdir(tmp_path / "cli" / "traj_000004")
  mem = run_benchmark.main(run_benchmark.parse_args(["--checkpoints", "3", "--steps", "1", "--payload_chars", "8"]))
  text = capsys.readouterr().out
  assert mem.passed and mem.writer_type == "InMemoryTrajectoryStore" and "load ms" in text
  temp = run_benchmark.FileTrajectoryStoreConfig().build()
  assert temp[2] and os.path.isdir(temp[2])
  temp[1].close()
  os.rmdir(temp[2])


# ---- process contexts --------------------------------------------------------------------------------
def _args(**kw):
  base = dict(discovery_id="", discovery_port=0, discovery_addrs="")
  base.update(kw)
  return types.SimpleNamespace(**base)


def test_names_resolve_per_platform(monkeypatch):
  assert local_context.resolve_discovery_address("door:12345") == "127.0.0.1:12345"
  assert k8s_context.resolve_discovery_address("door:12345") == "door-proc-0-0.door:12345"
  assert k8s_context.resolve_discovery_address("door:12345", jobset="run7") == "run7-door-0-0.run7:12345"
  for bad in ("door", "door:", ":x"):
    with pytest.raises(ValueError):
      k8s_context.resolve_discovery_address(bad)
  env = {"JOBSET_NAME": "myjobset", "REPLICATED_JOB_NAME": "worker", "JOB_INDEX": "0", "POD_INDEX": "2"}
  assert k8s_context.resolve_self_hostname(env) == "myjobset-worker-0-2.myjobset"
  del env["POD_INDEX"], env["JOB_INDEX"]
  with pytest.raises(ValueError, match="JOB_INDEX, POD_INDEX"):
    k8s_context.resolve_self_hostname(env)
  assert k8s_executor.pod_dns_name("js", "job", 1, 3) == "js-job-1-3.js"


def test_the_local_context_owns_its_discovery_listener():
  import socket
  with socket.socket() as s:
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
  heard = []
  with local_context.LocalProcessContext(_args(discovery_id="door", discovery_port=port)) as door:
    assert isinstance(door, rt_context.ProcessContext) and isinstance(door.ipc, local_context.LocalIpcContext)
    assert isinstance(door.dist, rt_context.DistContext) and door.dist.rank == int(os.environ.get("RANK", "0"))
    assert door.ipc.discovery.is_started() and door.ipc.discovery.port == port
    door.ipc.discovery.on_register(lambda host, p, meta: heard.append((host, p, meta)))
    with local_context.LocalProcessContext(_args(discovery_id="knocker", discovery_addrs=f"door:{port}")) as knocker:
      assert not knocker.ipc.discovery.is_started()          # no port: registers with others, serves nobody
      knocker.ipc.discovery.register(b"hello")
    import time
    for _ in range(100):
      if heard:
        break
      time.sleep(0.02)
  assert heard == [("knocker", 0, b"hello")] and not door.ipc.discovery.is_started()
  assert local_executor.LocalExecutor.context_cls is local_context.LocalProcessContext
  assert local_executor.LocalExecutor().run(lambda ctx, argv: (type(ctx).__name__, argv), ["--x"], _args()) == \
      ("LocalProcessContext", ["--x"])


def test_the_k8s_context_derives_rank_names_and_rendezvous_from_the_pod(monkeypatch):
  for var in ("RANK", "WORLD_SIZE", "MASTER_ADDR"):
    monkeypatch.delenv(var, raising=False)
  env = {"JOBSET_NAME": "run7", "REPLICATED_JOB_NAME": "trainer", "JOB_INDEX": "0", "POD_INDEX": "1",
         "JOB_COMPLETION_INDEX": "1", "TUNIX_NUM_NODES": "2", "TUNIX_GPUS_PER_NODE": "8", "LOCAL_RANK": "3"}
  ctx = k8s_context.K8sProcessContext(_args(discovery_id="trainer", discovery_addrs="rollout:7000"), environ=env)
  try:
    assert os.environ["RANK"] == "11" and os.environ["WORLD_SIZE"] == "16"
    assert os.environ["MASTER_ADDR"] == "run7-trainer-0-0.run7"
    assert ctx._resolve("rollout") == "run7-rollout-0-0.run7" and ctx._resolve("a.b.c") == "a.b.c"
    assert ctx._bind_host() == "0.0.0.0" and ctx.ipc.discovery._id == "run7-trainer-0-1.run7"
    assert isinstance(ctx.ipc, k8s_context.K8sIpcContext) and ctx.dist.world_size == 16
  finally:
    for var in ("RANK", "WORLD_SIZE", "MASTER_ADDR"):
      os.environ.pop(var, None)
  bare = k8s_context.K8sProcessContext(_args(discovery_id="solo"), environ={})
  assert bare.ipc.discovery._id == "solo" and bare._resolve("peer") == "peer"
  assert k8s_executor.K8sExecutor.context_cls is k8s_context.K8sProcessContext
