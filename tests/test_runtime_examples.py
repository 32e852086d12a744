"""The runtime examples run as they are documented: bodies under the launcher, door and knocker, the three-role toy
RL system over discovery and remote execution, and a worker driven through the transport example."""
import socket
import threading
import types

import pytest

from tunix_b200.experimental.common import datatypes
from tunix_b200.experimental.distributed.examples.basics import basic, door, flag, gpu, knocker
from tunix_b200.experimental.distributed.examples.rl import orchestrator, rollout, services, trainer
from tunix_b200.experimental.distributed.examples.worker_transport import remote_worker_server, transport
from tunix_b200.experimental.distributed.runtime import main as rt_main
from tunix_b200.experimental.distributed.runtime.contexts import local_context

EX = "tunix_b200.experimental.distributed.examples"


def free_port() -> int:
  with socket.socket() as s:
    s.bind(("127.0.0.1", 0))
    return s.getsockname()[1]


def ctx_args(**kw):
  base = dict(discovery_id="", discovery_port=0, discovery_addrs="")
  base.update(kw)
  return types.SimpleNamespace(**base)


def test_basic_and_flag_bodies_run_under_the_launcher(capsys):
  rt_main.main(["prog", f"--process_main={EX}.basics.basic.main"])
  rt_main.main(["prog", f"--process_main={EX}.basics.flag.main", "--message=hi there"])
  assert capsys.readouterr().out.splitlines()[-2:] == ["hello world", "hi there"]
  assert basic.main and flag.main


def test_door_hears_the_knocker():
  port = free_port()
  result = {}

  def run_door():
    with local_context.LocalProcessContext(ctx_args(discovery_id="door", discovery_port=port)) as ctx:
      result["heard"] = door.main(ctx, ["--wait_s=20"])
  t = threading.Thread(target=run_door)
  t.start()
  with local_context.LocalProcessContext(ctx_args(discovery_id="knocker", discovery_addrs=f"door:{port}")) as ctx:
    knocker.main(ctx, ["--say=open up"])
  t.join(30)
  assert result["heard"] == "knocker knocked and said: open up"
  with local_context.LocalProcessContext(ctx_args(discovery_id="lonely", discovery_port=free_port())) as ctx:
    with pytest.raises(SystemExit, match="nobody knocked"):
      door.main(ctx, ["--wait_s=0.05"])


def test_the_gpu_body_joins_a_group_and_describes_where_it_runs(monkeypatch):
  monkeypatch.setenv("MASTER_PORT", str(free_port()))
  for var in ("RANK", "WORLD_SIZE"):
    monkeypatch.delenv(var, raising=False)
  with local_context.LocalProcessContext(ctx_args()) as ctx:
    line = gpu.main(ctx, [])
  assert line.startswith("rank 0 of 1 (") and ("cuda:" in line or "no GPU visible" in line)


def test_arithmetic_prompts_are_evaluated_without_eval():
  assert services.evaluate("3 + 4") == 7 and services.evaluate("2 * 10") == 20 and services.evaluate("0 - 9") == -9
  for hostile in ("__import__('os').system('true')", "1 + 2 + 3", "2 ** 99", "a + 1", "1.5 + 1"):
    with pytest.raises((ValueError, SyntaxError)):
      services.evaluate(hostile)
  r = services.RolloutService("a", seed=1)
  assert all(abs(int(r.generate("5 + 5")[2:]) - 10) <= 1 for _ in range(20)) and r.served == 20
  t = services.TrainerService()
  assert t.train("1 + 1", "= 2") == "step 1: accuracy 1.00" and t.train("1 + 1", "= 3") == "step 2: accuracy 0.50"
  assert services.parse_announcement(services.announce("rollout", 5, "a")) == \
      {"service_type": "rollout", "server_port": 5, "server_id": "a"}
  with pytest.raises(ValueError, match="unknown service type"):
    services.parse_announcement(b'{"service_type": "critic"}')


def test_the_three_role_system_runs_under_one_launcher(caplog):
  rollout.stop.clear()
  disc, pa, pb, pt = free_port(), free_port(), free_port(), free_port()
  found = {}
  original = orchestrator.main

  def recording(ctx, argv):
    found["history"] = original(ctx, argv)
    return found["history"]
  orchestrator.main = recording
  try:
    rt_main.main([
        "prog",
        "--process", f"--process_main={EX}.rl.orchestrator.main", "--discovery_id=orchestrator",
        f"--discovery_port={disc}", "--max_train_step=6", "--wait_s=30",
        "--process", f"--process_main={EX}.rl.rollout.main", "--discovery_id=rollout-a",
        f"--discovery_addrs=orchestrator:{disc}", "--server_id=a", f"--server_port={pa}",
        "--process", f"--process_main={EX}.rl.rollout.main", "--discovery_id=rollout-b",
        f"--discovery_addrs=orchestrator:{disc}", "--server_id=b", f"--server_port={pb}", "--seed=5",
        "--process", f"--process_main={EX}.rl.trainer.main", "--discovery_id=trainer",
        f"--discovery_addrs=orchestrator:{disc}", f"--server_port={pt}"])
  finally:
    orchestrator.main = original
    rollout.stop.clear()
  history = found["history"]
  assert len(history) == 6 and history[-1].startswith("[5] ") and "[trainer] step 6: accuracy" in history[-1]
  assert all("-> [a] = " in line or "-> [b] = " in line for line in history)
  assert trainer.main


def test_a_missing_worker_ends_the_orchestrator_with_a_message():
  with local_context.LocalProcessContext(ctx_args(discovery_id="o", discovery_port=free_port())) as ctx:
    with pytest.raises(SystemExit, match="0 of 2 rollout workers, trainer missing"):
      orchestrator.main(ctx, ["--wait_s=0.05"])
  rollout.stop.clear()


def test_a_worker_in_another_server_is_driven_through_the_worker_interface():
  remote_worker_server.stop.clear()
  port = free_port()

  def serve():
    with local_context.LocalProcessContext(ctx_args()) as ctx:
      remote_worker_server.main(ctx, ["--worker_id=remote-7", f"--port={port}"])
  t = threading.Thread(target=serve, daemon=True)
  t.start()
  w = None
  for _ in range(200):
    try:
      w = transport.RemoteWorker(f"grpc://127.0.0.1:{port}")
      w.heartbeat()
      break
    except Exception:  # noqa: BLE001 - the server is still starting
      import time
      time.sleep(0.05)
  try:
    S = datatypes.WorkerState
    assert w.state == S.PENDING and w.info().worker_id == "remote-7" and w.info().roles == frozenset({"rollout"})
    w.initialize(); w.compile(); w.start()
    assert w.state == S.READY and isinstance(w.heartbeat(), datatypes.HealthReport)
    w.stop()
    assert w.state == S.STOPPED
    with pytest.raises(Exception, match="Invalid transition from STOPPED"):
      w.call("initialize")                                     # the remote error arrives with its message
  finally:
    remote_worker_server.stop.set()
    t.join(10)
    remote_worker_server.stop.clear()


def test_remote_invocation_demo_awaits_and_polls():
  from tunix_b200.experimental.distributed.examples.vllm_rollout import remote
  with local_context.LocalProcessContext(ctx_args()) as ctx:
    out = remote.main(ctx, [])
  assert out["squares"] == [9, 16, 25] and out["worker_id"].startswith("worker-")


@pytest.mark.timeout(300)
def test_generation_load_is_spread_over_discovered_rollout_workers():
  from tunix_b200.experimental.distributed.examples.vllm_rollout import orchestrator as load, rollout as load_rollout
  load_rollout.stop.clear()
  disc = free_port()
  out = {}
  original = load.main

  def recording(ctx, argv):
    out["summary"] = original(ctx, argv)
    return out["summary"]
  load.main = recording
  worker = lambda wid: ["--process", f"--process_main={EX}.vllm_rollout.rollout.main", f"--discovery_id=rollout-{wid}",   # noqa: E731
                        f"--discovery_addrs=orchestrator:{disc}", f"--worker_id={wid}", "--port=0", "--max_seq_len=64",
                        "--max_batch=8"]
  try:
    rt_main.main(["prog", "--process", f"--process_main={EX}.vllm_rollout.orchestrator.main",
                  "--discovery_id=orchestrator", f"--discovery_port={disc}", "--num_requests=12", "--concurrency=4",
                  "--max_tokens=6", "--wait_s=120", *worker("a"), *worker("b")])
  finally:
    load.main = original
    load_rollout.stop.clear()
  s = out["summary"]
  assert not s["failures"], s["failures"]
  assert sum(s["requests"].values()) == 12 and set(s["requests"]) == {"a", "b"}
  assert 12 <= sum(s["tokens"].values()) <= 72 and s["requests_per_s"] > 0
  m = load.RequestStatsMonitor(log_interval_seconds=3600)
  m.record_request("w", 5); m.record_request("w", 7)
  assert m.total_requests == 2 and m.summary()["tokens"] == {"w": 12}
  assert not m.maybe_log_summary() and m.maybe_log_summary(force=True)
  assert load.RolloutSpec.from_announcement("10.0.0.5", b"a|50081|tiny") == load.RolloutSpec("a", "grpc://10.0.0.5:50081", "tiny")
