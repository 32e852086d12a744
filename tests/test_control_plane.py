"""Control plane on CPU with injected failures: lifecycle ordering, health deadlines with a fake
clock, registry, startup validation, remote execution, weight-sync rounds and their failure
states. All failures are made on the host: a worker that raises, a reply that is dropped, a
transfer that does not return in time."""
import os
import asyncio
import threading
import time

import pytest
import torch

from tunix_b200.experimental.common import datatypes
from tunix_b200.experimental.orchestrator import (health_monitor, lifecycle, peer_memory_handler, startup_validation,
                                                  weight_sync, weight_sync_coordinator as wsc, worker_registry)
from tunix_b200.experimental.worker import mock_worker, remote_execution as rx, traffic_controller

S = datatypes.WorkerState


def test_state_machine_and_mock_worker():
  w = mock_worker.MockWorker("w0", {"trainer"})
  assert w.state == S.PENDING
  with pytest.raises(RuntimeError, match="Invalid transition"):
    w.state = S.SYNCING
  w.initialize(); w.compile(); w.start()
  w.state = S.SYNCING
  w.state = S.READY
  w.stop()
  with pytest.raises(RuntimeError):
    w.state = S.READY
  assert w.call_counts == {"initialize": 1, "compile": 1, "start": 1, "stop": 1}


def test_lifecycle_phases_are_barriers_and_shutdown_is_best_effort():
  log = []
  reg = worker_registry.WorkerRegistry()
  for i in range(4):
    reg.register(mock_worker.MockWorker(f"w{i}", {"rollout" if i else "trainer"}, log=log, fail_stop=(i == 2)))
  with pytest.raises(ValueError, match="duplicate"):
    reg.register(mock_worker.MockWorker("w1", {"rollout"}))
  with pytest.raises(ValueError, match="no roles"):
    reg.register(mock_worker.MockWorker("w9", set()))
  drv = lifecycle.LifecycleDriver(reg)
  drv.bring_up(None)
  phases = [e.split(":")[1] for e in log]
  assert phases == ["initialize"] * 4 + ["compile"] * 4 + ["start"] * 4
  assert len(reg.group("rollout")) == 3 and reg.roles() == {"trainer", "rollout"}
  with pytest.raises(lifecycle.LifecycleError) as ei:
    drv.shutdown()
  assert [w for w, _ in ei.value.failures] == ["w2"]
  assert all(w.state == S.STOPPED for w in reg.workers())           # every worker was still stopped
  reg2 = worker_registry.WorkerRegistry()
  reg2.register(mock_worker.MockWorker("a", {"trainer"}, fail_in={"compile"}))
  reg2.register(mock_worker.MockWorker("b", {"rollout"}))
  with pytest.raises(lifecycle.LifecycleError, match="compile failed for 1 worker"):
    lifecycle.LifecycleDriver(reg2).bring_up(None)
  assert reg2.get("b").call_counts["start"] == 0                       # later phases did not run


def test_health_monitor_deadlines_with_fake_clock():
  now = [0.0]
  reg = worker_registry.WorkerRegistry()
  a, b = mock_worker.MockWorker("a", {"rollout"}), mock_worker.MockWorker("b", {"rollout"})
  for w in (a, b):
    reg.register(w); w.initialize(); w.start()
  b.heartbeat = lambda: (_ for _ in ()).throw(ConnectionError("gone"))
  with health_monitor.HealthMonitor(reg, clock=lambda: now[0], state_deadlines_s={S.SYNCING: 10.0}) as mon:
    rep = mon.poll()
    assert rep["a"].state == S.READY and rep["b"].state == S.ERROR and "gone" in rep["b"].last_error
    assert mon.unhealthy() == ["b"] and mon.overdue() == []
    a.state = S.SYNCING
    mon.poll(); now[0] = 9.0
    assert mon.overdue() == []
    now[0] = 11.0; mon.poll()
    od = mon.overdue()
    assert [(o.worker_id, o.state) for o in od] == [("a", "SYNCING")] and od[0].elapsed_s == 11.0
    a.state = S.READY; mon.poll()
    assert mon.overdue() == []
    reg.unregister("b"); mon.poll()
    assert mon.unhealthy() == []


def test_startup_validation_collects_everything():
  class A: num_generations = 3; max_response_length = 0; algo_variant = "grpo"
  class T: mini_batch_size = 8; train_micro_batch_size = 3; rollout_micro_batch_size = None; compute_logps_micro_batch_size = 4
  reg = worker_registry.WorkerRegistry()
  with pytest.raises(startup_validation.StartupValidationError) as ei:
    startup_validation.validate_startup(reg, A, T, validators=(startup_validation.RunGeometryValidator(),
                                                                startup_validation.RoleCoverageValidator()))
  msgs = "\n".join(ei.value.errors)
  assert "max_response_length" in msgs and "num_generations (group_size) 3" in msgs and "train_micro_batch_size 3" in msgs
  assert "role 'actor'" in msgs and len(ei.value.errors) == 5


def test_traffic_controller_gates_admission():
  async def run():
    tc = traffic_controller.TrafficController()
    async def job(): await asyncio.sleep(0.05); return 1
    t1 = asyncio.create_task(job())
    assert tc.try_admit(t1) and tc.get_active_tasks() == [t1]
    tc.transition_to_syncing()
    t2 = asyncio.create_task(job())
    assert not tc.try_admit(t2) and not tc.is_admission_open()
    await tc.drain(1.0)
    assert tc.get_active_tasks() == [] and t1.result() == 1
    with pytest.raises(asyncio.CancelledError):
      await t2
    assert tc.reopen() and tc.is_admission_open()
    t3 = asyncio.create_task(asyncio.sleep(10)); tc.try_admit(t3)
    assert tc.stop_and_cancel_all() == [t3] and not tc.reopen()
    with pytest.raises(RuntimeError, match="Cannot transition"):
      tc.transition_to_syncing()
  asyncio.run(run())


def test_remote_execution_inprocess_routing_and_errors():
  class W:
    def __init__(self, k): self.k = k; self.seen = []
    def mul(self, x): self.seen.append(x); return x * self.k
    async def amul(self, x): await asyncio.sleep(0.005 * x); return x * self.k
    def boom(self): raise KeyError("k")
    def unpicklable(self): return threading.Lock()
  hs = [rx.remote(W).remote(k) for k in (1, 10)]
  assert hs[0].submit("mul", 3) == 3
  with pytest.raises(RuntimeError, match=r"RemoteExecutionError \[KeyError\]"):
    hs[0].submit("boom")
  with pytest.raises(RuntimeError, match="not found"):
    hs[0].submit("nope")
  with pytest.raises(ValueError, match="reserved"):
    rx.ExecutionRequest(method_name="mul", kwargs={"request_id": 1})
  r = rx.ExecutionResponse(result=threading.Lock())
  assert rx.ExecutionResponse.deserialize(r.serialize()).error_type == "ExecutionResponseSerializationError"
  pool = rx.RoutingActorPool(hs)
  assert [pool.submit("mul", 1) for _ in range(4)] == [1, 10, 1, 10]                    # round robin
  assert {pool.submit("mul", 1, route_key="user-7") for _ in range(5)} in ({1}, {10})   # sticky
  pool2 = rx.RoutingActorPool(hs, router=lambda actors, m, a, k: actors[1])
  assert pool2.submit("mul", 2) == 20

  async def stream():
    out, errs = [], []
    async with pool.execution_session([(f"t{i}", "amul", (i,), {}) for i in range(4)]) as s:
      await s.submit("bad", "boom")
      async for res, exc in s.as_completed():
        (errs if exc else out).append(exc or res)
    return sorted(out), errs
  out, errs = asyncio.run(stream())
  assert out == [0, 2, 10, 30] and len(errs) == 1 and "KeyError" in str(errs[0])

  @rx.remote
  def add(a, b): return a + b
  assert add.remote(2, 3) == 5


# ---- weight sync ---------------------------------------------------------------------------------
class FakeSource:
  def __init__(self, handler, fail_prepare=False):
    self.handler, self.fail_prepare = handler, fail_prepare
    self.weights = {"w": torch.zeros(4, 3), "b": torch.zeros(3)}
    self.unit = weight_sync.WorkUnitId(job_name="trainer")
    self.released = 0
  def info(self): return datatypes.WorkerInfo(worker_id="trainer0", roles=frozenset({"trainer"}))
  async def prepare_weight_sync(self, req=None, **kw):
    if self.fail_prepare:
      raise RuntimeError("D2H failed")
    self.handler.attach(self.unit, {k: v.clone() for k, v in self.weights.items()})
    return [peer_memory_handler.manifest_of(self.unit, self.weights)]
  async def release_weight_sync(self, req=None, **kw):
    self.released += 1


class FakeDest:
  """Follows the destination contract: staging only in weight_sync, atomic publish in post."""
  def __init__(self, handler, wid, fail=None, lose_reply=None):
    self.handler, self.wid, self.fail, self.lose_reply = handler, wid, fail or set(), lose_reply or set()
    self.serving = {"w": torch.full((4, 3), -1.0), "b": torch.full((3,), -1.0)}
    self.staging = {k: torch.zeros_like(v) for k, v in self.serving.items()}
    self.unit = weight_sync.WorkUnitId(job_name="rollout", job_replica_id=wid)
    self.tracker = wsc.WorkerRoundTracker()
    self.admitting, self.version, self.calls = True, 0, []
  def info(self): return datatypes.WorkerInfo(worker_id=self.wid, roles=frozenset({"rollout"}))
  async def bind_weight_sync(self): self.handler.attach(self.unit, self.staging)
  async def get_weight_sync_metadata(self): return [peer_memory_handler.manifest_of(self.unit, self.staging)]
  async def get_weight_sync_status(self): return self.tracker.report()
  async def _phase(self, name, phase, req, work):
    self.calls.append(name)
    if name in self.fail:
      raise RuntimeError(f"{self.wid} cannot {name}")
    if self.tracker.admit(req, phase):
      work()
      self.tracker.complete(req, phase)
    if name in self.lose_reply:
      raise ConnectionError("reply lost")
  async def pre_weight_sync(self, req=None):
    await self._phase("pre_weight_sync", "prepared", req, lambda: setattr(self, "admitting", False))
  async def weight_sync(self, req=None):
    await self._phase("weight_sync", "h2d_done", req, lambda: None)
  async def post_weight_sync(self, req=None):
    def publish():
      self.serving = {k: v.clone() for k, v in self.staging.items()}
      self.version, self.admitting = req.policy_version, True
    await self._phase("post_weight_sync", "committed", req, publish)
  async def abort_weight_sync(self, req=None):
    await self._phase("abort_weight_sync", "aborted", req, lambda: setattr(self, "admitting", True))


def make_round(**dest_kw):
  h = peer_memory_handler.InProcessHandler()
  src = FakeSource(h)
  dests = [FakeDest(h, f"r{i}", **{k: (v[i] if isinstance(v, list) else v) for k, v in dest_kw.items()}) for i in range(2)]
  co = wsc.WeightSyncCoordinator(h, sources=[src], destinations=dests, timeouts=wsc.PhaseTimeouts(transfer=0.5))
  return h, src, dests, co


def test_weight_sync_preflight_catches_name_and_shape_mismatches_before_any_downtime():
  h, src, dests, co = make_round()
  dests[1].serving = {"w": torch.full((4, 3), -1.0), "bias": torch.full((3,), -1.0)}        # a misspelt name
  dests[1].staging = {k: torch.zeros_like(v) for k, v in dests[1].serving.items()}
  res = asyncio.run(co.sync(1, raise_on_failure=False))
  assert res.state == wsc.RoundState.ABORTED and not co.poisoned
  text = " ".join(res.failures)
  assert "destination units disagree" in text or "'bias' has no source counterpart" in text
  assert all("pre_weight_sync" not in d.calls for d in dests) and all(d.admitting for d in dests)
  assert src.released == 1
  m_src = wsc.Manifest("source", [peer_memory_handler.manifest_of(src.unit, {"w": torch.zeros(4, 3)})])
  m_dst = wsc.Manifest("destination", [peer_memory_handler.manifest_of(dests[0].unit, {"w": torch.zeros(4, 3).half()})])
  assert m_src.differences(m_dst) == ["preflight: 'w' item_size differs: source 4, destination 2"]
  m_dst2 = wsc.Manifest("destination", [peer_memory_handler.manifest_of(dests[0].unit, {"w": torch.zeros(2, 3)})])
  assert "global shape differs" in m_src.differences(m_dst2)[0]


def test_weight_sync_commits_and_versions_advance():
  h, src, dests, co = make_round()
  src.weights["w"].fill_(2.0)
  res = asyncio.run(co.sync(1))
  assert res.success and res.state == wsc.RoundState.COMMITTED and co.last_committed_version == 1
  for d in dests:
    assert d.version == 1 and d.admitting and torch.equal(d.serving["w"], torch.full((4, 3), 2.0))
    assert d.calls == ["pre_weight_sync", "weight_sync", "post_weight_sync"]
  assert src.released == 1
  with pytest.raises(ValueError, match="does not advance"):
    asyncio.run(co.sync(1))
  src.weights["w"].fill_(3.0)
  assert asyncio.run(co.sync(2)).round_index == 2 and dests[0].serving["w"][0, 0] == 3.0


def test_pre_failure_rolls_back_and_keeps_serving_old_weights():
  h, src, dests, co = make_round(fail=[set(), {"pre_weight_sync"}])
  res = asyncio.run(co.sync(1, raise_on_failure=False))
  assert res.state == wsc.RoundState.ABORTED and co.poisoned is None
  assert all(d.admitting and d.version == 0 and d.serving["w"][0, 0] == -1.0 for d in dests)
  assert src.released == 1 and {r.phase for r in res.workers} == {"aborted"}
  with pytest.raises(wsc.WeightSyncError):
    asyncio.run(co.sync(2))                                   # same faulty worker: raises, still not poisoned
  assert co.poisoned is None


def test_lost_reply_is_reconciled_with_the_worker_report():
  h, src, dests, co = make_round(lose_reply=[{"weight_sync"}, {"post_weight_sync"}])
  assert asyncio.run(co.sync(1)).success and all(d.version == 1 for d in dests)


def test_partial_commit_poisons_the_coordinator():
  h, src, dests, co = make_round(fail=[set(), {"post_weight_sync"}])
  res = asyncio.run(co.sync(1, raise_on_failure=False))
  assert res.state == wsc.RoundState.PARTIALLY_COMMITTED
  assert dests[0].version == 1 and dests[1].version == 0
  bad = [r for r in res.workers if r.needs_restart]
  assert [r.worker_id for r in bad] == ["r1"] and bad[0].phase == "h2d_done"
  with pytest.raises(RuntimeError, match="poisoned"):
    asyncio.run(co.sync(2))
  co.reset_after_recovery()
  dests[1].fail = set()
  assert asyncio.run(co.sync(2)).success


def test_abort_failure_needs_restart_and_transfer_timeout_is_unknown():
  h, src, dests, co = make_round(fail=[{"weight_sync"}, {"abort_weight_sync"}])
  res = asyncio.run(co.sync(1, raise_on_failure=False))
  assert res.state == wsc.RoundState.FAILED_NEEDS_RESTART and co.poisoned
  h, src, dests, co = make_round()
  h.transfer = lambda *a, **k: time.sleep(2)                 # never answers within the deadline
  res = asyncio.run(co.sync(1, raise_on_failure=False))
  assert res.state == wsc.RoundState.UNKNOWN_TRANSFER_STATE
  assert src.released == 0 and all("abort_weight_sync" not in d.calls for d in dests)   # nothing released or aborted
  h, src, dests, co = make_round()
  src.fail_prepare = True
  res = asyncio.run(co.sync(1, raise_on_failure=False))
  assert res.state == wsc.RoundState.ABORTED and all(d.calls == [] for d in dests)        # no downtime at all


def test_round_tracker_rejects_stale_and_stray_phases():
  t = wsc.WorkerRoundTracker()
  rq = lambda u, rid=None: datatypes.WeightSyncRequest(policy_version=u, extra_config={"req_id": rid or f"r{u}", "uuid": u})
  with pytest.raises(wsc.StaleRoundError, match="cannot open a round"):
    t.admit(rq(1), "h2d_done")
  assert t.admit(rq(1), "prepared"); t.complete(rq(1), "prepared")
  assert not t.admit(rq(1), "prepared")                        # duplicate delivery
  assert t.admit(rq(1), "h2d_done"); t.complete(rq(1), "h2d_done")
  with pytest.raises(wsc.StaleRoundError, match="never be reused"):
    t.admit(rq(1, "other"), "committed")
  with pytest.raises(wsc.StaleRoundError, match="cannot open"):
    t.admit(rq(3), "committed")                                # stray mid-round phase of a future round
  assert t.admit(rq(2), "aborted"); t.complete(rq(2), "aborted")
  with pytest.raises(wsc.StaleRoundError, match="already aborted"):
    t.admit(rq(2), "committed")
  with pytest.raises(wsc.StaleRoundError, match="rejected"):
    t.admit(rq(1), "committed")                                # late retry from an older round
  assert t.report()["phase"] == "aborted" and t.report()["uuid"] == 2


def test_manifest_validation():
  with pytest.raises(ValueError, match="one mesh axis for two tensor"):
    weight_sync.TensorMetadata(name="w", shape=(2, 2), mesh_shape=(1, 1), layout=(1, 0), item_size=2, sharding_spec=("x", "x"))
  with pytest.raises(ValueError, match="rank"):
    weight_sync.TensorMetadata(name="w", shape=(2, 2), mesh_shape=(1,), layout=(1, 0), item_size=2)
  with pytest.raises(NotImplementedError):
    datatypes.WeightSyncMetadata(transfer_mode="fs")
  h = peer_memory_handler.InProcessHandler()
  u1, u2 = weight_sync.WorkUnitId(job_name="a"), weight_sync.WorkUnitId(job_name="b")
  h.register_work_unit(peer_memory_handler.manifest_of(u1, {"w": torch.zeros(2, 2)})); h.attach(u1, {"w": torch.zeros(2, 2)})
  h.register_work_unit(peer_memory_handler.manifest_of(u2, {"w": torch.zeros(3, 2)})); h.attach(u2, {"w": torch.zeros(3, 2)})
  r = h.transfer([u1], [u2], req_id="x")
  assert not r.success and "shape mismatch" in r.message


# ---- the whole loop in one process ---------------------------------------------------------------
@pytest.mark.parametrize("transport", ["in_process", "host_staged"])
def test_rl_program_end_to_end_with_workers_and_weight_sync(transport):
  """`host_staged`: the same program with the weights crossing real TCP sockets between a source endpoint
  (the trainer worker's) and a destination endpoint (the sampler's), commanded by the coordinator's handler."""
  from tests.test_rl_grpo import ToyTokenizer, toy_model
  from tunix_b200 import optim
  from tunix_b200.common.configs import TrainingConfig
  from tunix_b200.experimental.orchestrator import (algorithm_adapter, batch_assembly, orchestrator as orch_lib,
                                                    rl_program)
  from tunix_b200.experimental.rollout import manager as manager_lib, native_sampler_adapter
  from tunix_b200.experimental.train import peft_trainer_v2
  from tunix_b200.experimental.worker import inference_worker, rollout_worker, trainer_worker
  from tunix_b200.rl import function_registry
  from tunix_b200.rl.grpo.grpo_learner import GRPOConfig
  from tunix_b200.rollout import EngineConfig

  tok = ToyTokenizer()
  actor, rollout_model, ref = toy_model(), toy_model(), toy_model()
  endpoints = []
  if transport == "in_process":
    handler = source_side = destination_side = peer_memory_handler.InProcessHandler()
  else:
    from tunix_b200.experimental.orchestrator import host_staged_handler as hs
    source_side, destination_side = hs.HostStagedEndpoint(), hs.HostStagedEndpoint()
    endpoints = [source_side, destination_side]
    handler = hs.HostStagedHandler(timeout_s=30)
  algo_cfg = GRPOConfig(num_generations=2, beta=0.04)
  loss = function_registry.get_policy_loss_fn("grpo")

  def make_trainer():
    t = peft_trainer_v2.PeftTrainerV2(actor, optim.adamw(1e-2), TrainingConfig(eval_every_n_steps=100, pbar_description=None))
    t.with_loss_fn(lambda model, train_example: loss(model, train_example.to_tensors(), algo_config=algo_cfg,
                                                     pad_id=0, eos_id=2), has_aux=True)
    t.with_gen_model_input_fn(lambda x: {"train_example": x})
    return t
  tw = trainer_worker.TrainerWorker(make_trainer, worker_id="t0", handler=source_side)
  sampler = native_sampler_adapter.NativeSamplerAdapter(rollout_model, tok, handler=destination_side, worker_id="r0",
                                                        engine_config=EngineConfig(page_size=4, max_batch=8, max_seq_len=32))
  if endpoints:
    handler.register_endpoint(tw.work_unit, source_side.address)
    handler.register_endpoint(sampler.work_unit, destination_side.address)
  rw = rollout_worker.RolloutWorker(lambda: manager_lib.RolloutManager(sampler=sampler, tokenizer=tok, chat_parser=None),
                                    worker_id="r0")
  iw = inference_worker.InferenceWorker({"reference": ref}, worker_id="i0")
  co = wsc.WeightSyncCoordinator(handler, sources=[tw], destinations=[rw])
  orch = orch_lib.ClusterOrchestrator(weight_sync_coordinator=co)
  for w in (tw, rw, iw):
    orch.register_worker(w)
  before = {n: p.detach().clone() for n, p in rollout_model.named_parameters()}
  algo = algorithm_adapter.GRPOAdapter(group_size=2, mini_batch_size=2, beta_kl=0.04)
  prog = rl_program.StandardRLProgram(
      algo, reward_fns=[lambda item: float(len(item.completion_tokens)) / 8.0 + 0.1 * item.pair_index],
      assembler=batch_assembly.GRPOTrainExampleAssembler(batch_size=2, max_prompt_length=8, max_response_length=8, pad_id=0),
      max_staleness=1)
  ds = [{"prompt": f"alpha beta {w}", "generation_kwargs": {"max_generation_steps": 8, "temperature": 1.0, "seed": i}}
        for i, w in enumerate(["gamma", "delta", "eps", "zeta", "eta", "theta"])]
  with orch:
    reports, overdue, bad = orch.poll_health()
    assert {r.state for r in reports.values()} == {S.READY} and not overdue and not bad
    orch.run_program(prog, ds, num_steps=2)
  assert [r.policy_version for r in prog.history] == [1, 2] and prog.history[0].num_rollouts == 4
  assert co.last_committed_version == 2 and sampler.policy_version == 2
  assert tw.trainer.train_steps == 2
  changed = [n for n, p in rollout_model.named_parameters() if not torch.equal(p, before[n])]
  assert changed                                                     # the rollout model received the new weights
  for n, p in rollout_model.named_parameters():
    torch.testing.assert_close(p, dict(actor.named_parameters())[n])
  assert all(w.state == S.STOPPED for w in (tw, rw, iw))
  if endpoints:
    assert source_side.served["fetch"] == 2 and destination_side.served["pull"] == 2
  for ep in endpoints:
    ep.close()


def test_remote_execution_over_grpc_loopback():
  """A worker object served by the gRPC `RemoteExecutionServer` on 127.0.0.1 and driven through a
  `GrpcRemoteActorHandle`: unary calls, remote errors, and the dispatch / long-poll pair."""
  grpc = pytest.importorskip("grpc")

  class Worker:
    def __init__(self): self.calls = 0
    def scale(self, x, k=2): self.calls += 1; return [v * k for v in x]
    async def slow_add(self, a, b): await asyncio.sleep(0.01); return a + b
    def fail(self): raise ValueError("nope")

  w = Worker()
  server = rx.GrpcRemoteExecutionServer(w)
  server.start_serving(port=0)                      # port 0: the OS picks a free one
  assert server.port and server.port > 0
  handle = rx.ActorHandle.from_address(f"grpc://127.0.0.1:{server.port}")
  try:
    assert handle.submit("scale", [1, 2, 3], k=3) == [3, 6, 9] and w.calls == 1
    with pytest.raises(RuntimeError, match=r"RemoteExecutionError \[ValueError\]"):
      handle.submit("fail")

    async def session():
      assert await handle.asubmit("slow_add", 2, 5) == 7
      rid = await handle.dispatch_task("job-1", "scale", [4], k=5)
      assert rid == "job-1"
      got = []
      for _ in range(20):
        got += await handle.poll_responses(timeout_s=0.5, max_items=4)
        if got:
          break
      assert [r.request_id for r in got] == ["job-1"] and got[0].unwrap() == [20]
      await handle.close()
    asyncio.run(session())
  finally:
    server.shutdown()


def test_host_staged_transport_between_processes():
  """`host_staged_handler`: a source and two destinations in their own OS processes, the handler in this one.
  Bytes arrive exactly (same dtype) or converted (fp32 staging), stale generations and shape mismatches are
  refused, an unreachable destination is a known failure."""
  import subprocess
  import sys
  import torch
  from tests import _host_staged_worker as w
  from tunix_b200.experimental.orchestrator import host_staged_handler as hs, peer_memory_handler as pmh, weight_sync as ws
  here = os.path.dirname(os.path.abspath(__file__))
  procs = []

  def spawn(role, unit, generation=0):
    p = subprocess.Popen([sys.executable, os.path.join(here, "_host_staged_worker.py"), role, unit, str(generation)],
                         stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True)
    procs.append(p)
    return ("127.0.0.1", int(p.stdout.readline()))

  try:
    src, same, wide = (ws.WorkUnitId("trainer", "t0", 0), ws.WorkUnitId("rollout", "r0", 0),
                       ws.WorkUnitId("rollout", "r1", 1))
    addr = {src: spawn("source", hs.unit_key(src), 5), same: spawn("same", hs.unit_key(same)),
            wide: spawn("wide", hs.unit_key(wide))}
    handler = hs.HostStagedHandler(addr, timeout_s=30)
    want = w.tensors(7, torch.bfloat16)
    handler.register_work_unit(pmh.manifest_of(src, want))
    assert not handler.transfer([src], [same], "r1", 5).success          # destination never registered
    handler.register_work_unit(pmh.manifest_of(same, w.tensors(0, torch.bfloat16)))
    handler.register_work_unit(pmh.manifest_of(wide, w.tensors(0, torch.float32)))
    stale = handler.transfer([src], [same], "r2", generation=4)
    assert not stale.success and "generation" in stale.message
    done = handler.transfer([src], [same, wide], "r3", generation=5)
    assert done.success and "2 destination" in done.message, done.message
    # the bf16 destination holds the source's bytes; the fp32 one holds the converted values
    digest = lambda a, u: hs.call(a, {"op": "checksum", "unit": hs.unit_key(u)})["sha256"]   # noqa: E731
    assert digest(addr[same], same) == digest(addr[src], src)
    import hashlib
    expect = hashlib.sha256()
    for n in sorted(want):
      expect.update(n.encode())
      expect.update(want[n].float().contiguous().view(-1).view(torch.uint8).numpy().tobytes())
    assert digest(addr[wide], wide) == expect.hexdigest()
    # a manifest that disagrees on a shape is caught before anything moves
    bad = dict(w.tensors(0, torch.bfloat16))
    bad["layers.0.w"] = torch.zeros(16, 47)
    handler.register_work_unit(pmh.manifest_of(same, bad))
    assert "shape mismatch" in handler.transfer([src], [same], "r4", 5).message
    # an endpoint nobody listens on: failure, not an unknown outcome
    handler.register_work_unit(pmh.manifest_of(same, w.tensors(0, torch.bfloat16)))
    handler.register_endpoint(same, ("127.0.0.1", 1))
    gone = handler.transfer([src], [same], "r5", 5)
    assert not gone.success and "unreachable" in gone.message
  finally:
    for p in procs:
      p.stdin.close()
      p.wait(timeout=10)
