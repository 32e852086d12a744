"""Workers of the control plane one by one: the lifecycle every worker shares, the inference worker's log-probs and
scores against direct model calls, the trainer worker's replies, error state and weight-sync staging, the rollout
worker's destination phases, and the admission gate."""
import asyncio

import numpy as np
import pytest
import torch

from tests.test_rl_grpo import toy_model
from tunix_b200.experimental.common import datatypes
from tunix_b200.experimental.worker import (inference_worker, mock_worker, rollout_worker, traffic_controller,
                                            trainer_worker)
from tunix_b200.rl import common as rl_common

S = datatypes.WorkerState


# ---- lifecycle ------------------------------------------------------------------------------------
def test_the_state_machine_allows_the_documented_paths_only():
  w = mock_worker.MockWorker("m0", ["rollout"])
  assert w.state == S.PENDING and w.heartbeat().state == S.PENDING and w.info().roles == frozenset({"rollout"})
  with pytest.raises(RuntimeError, match="Invalid transition from PENDING to READY"):
    w.state = S.READY
  w.initialize()
  assert w.state == S.INITIALIZING
  w.compile()
  w.start()
  assert w.state == S.READY and w.call_counts == {"initialize": 1, "compile": 1, "start": 1}
  w.state = S.SYNCING
  w.state = S.SYNCING                                 # same state: no-op
  w.state = S.READY
  w.stop()
  assert w.state == S.STOPPED
  with pytest.raises(RuntimeError, match="Invalid transition from STOPPED"):
    w.state = S.READY
  for state in S:
    assert state.can_transition_to(S.ERROR) == (state not in (S.STOPPED, S.ERROR))


def test_the_mock_worker_logs_order_and_fails_where_told():
  log = []
  a = mock_worker.MockWorker("a", ["x"], log=log)
  b = mock_worker.MockWorker("b", ["x"], log=log, fail_in=["compile"])
  for w in (a, b):
    w.initialize()
  a.compile()
  with pytest.raises(RuntimeError, match="b failed in compile"):
    b.compile()
  assert log == ["a:initialize", "b:initialize", "a:compile", "b:compile"]
  with pytest.raises(RuntimeError, match="refused to stop"):
    mock_worker.MockWorker("c", ["x"], fail_stop=True).stop()


# ---- inference worker -----------------------------------------------------------------------------
def _batch(seed=0, B=5, P=6, C=7):
  g = np.random.default_rng(seed)
  p = g.integers(3, 60, (B, P))
  c = g.integers(3, 60, (B, C))
  p[0, :2] = 0                                        # left padding
  c[1, 4], c[1, 5:] = 2, 0                            # EOS then padding
  c[2, 3:] = 0                                        # cut off without EOS
  return p, c


class Scorer(torch.nn.Module):
  """Per-token score = the token id (as a float), so that the picked position is visible in the value."""

  def __init__(self):
    super().__init__()
    self.w = torch.nn.Parameter(torch.ones(1))

  def forward(self, ids, positions, cache, mask):
    return (ids.float() * self.w)[..., None], None


def test_logprobs_match_a_direct_call_with_temperature_and_in_chunks():
  ref = toy_model(seed=3)
  p, c = _batch()
  whole = inference_worker.InferenceWorker({"reference": ref})
  whole.initialize()
  req = datatypes.LogprobsRequest(request_id="q1", prompt_tokens=p, completion_tokens=c, temperature=0.7)
  got = whole.per_token_logps(request=req)
  want = rl_common.compute_per_token_logps(ref, torch.from_numpy(p), torch.from_numpy(c), 0, 2, stop_gradient=True,
                                           temperature=0.7)
  want = want[0] if isinstance(want, tuple) else want
  assert got.request_id == "q1" and got.per_token_logps.shape == c.shape and got.per_token_logps.dtype == np.float32
  np.testing.assert_allclose(got.per_token_logps, want.numpy(), atol=1e-5)
  cold = whole.per_token_logps(request=datatypes.LogprobsRequest(request_id="q", prompt_tokens=p, completion_tokens=c,
                                                                 temperature=1.0))
  assert np.abs(cold.per_token_logps - got.per_token_logps).max() > 1e-3
  chunked = inference_worker.InferenceWorker({"reference": ref}, micro_batch_size=2)   # 5 rows: 2 + 2 + 1
  np.testing.assert_allclose(chunked.compute_logps(req).per_token_logps, got.per_token_logps, atol=1e-5)

  class Example:                                        # anything with prompt_ids / completion_ids works too
    prompt_ids, completion_ids = torch.from_numpy(p), torch.from_numpy(c)
  np.testing.assert_allclose(whole.per_token_logps(Example, temperature=0.7).per_token_logps, got.per_token_logps, atol=1e-5)


def test_bad_requests_are_refused_and_show_up_in_the_heartbeat():
  w = inference_worker.InferenceWorker({"reference": toy_model()}, worker_id="i0")
  w.initialize()
  p, c = _batch()
  with pytest.raises(KeyError, match="no model hosted for role 'actor'"):
    w.per_token_logps(request=datatypes.LogprobsRequest(prompt_tokens=p, completion_tokens=c, temperature=1.0, model_role="actor"))
  assert "KeyError" in w.heartbeat().last_error and w.heartbeat().state == S.READY
  with pytest.raises(ValueError, match="strictly positive"):
    w.per_token_logps(request=datatypes.LogprobsRequest(prompt_tokens=p, completion_tokens=c, temperature=0.0))
  with pytest.raises(KeyError, match="'reward'"):
    w.score(request=datatypes.ScoreRequest(prompt_tokens=p, completion_tokens=c))

  class Ragged:
    prompt_ids, completion_ids = [[1, 2], [3]], [[4], [5, 6]]
  with pytest.raises(ValueError, match="padded"):
    w.per_token_logps(Ragged)
  w.per_token_logps(request=datatypes.LogprobsRequest(prompt_tokens=p, completion_tokens=c, temperature=1.0))
  assert w.heartbeat().last_error is None               # a good call clears it
  assert w.info().roles == frozenset({"reference"}) and w.info().worker_id == "i0"
  w.stop()
  assert w.state == S.STOPPED


def test_scores_are_read_at_the_last_valid_completion_token():
  p, c = _batch()
  w = inference_worker.InferenceWorker({"reward": Scorer()}, micro_batch_size=2)
  w.initialize()
  out = w.score(request=datatypes.ScoreRequest(request_id="s1", prompt_tokens=p, completion_tokens=c))
  assert out.request_id == "s1" and out.scores.shape == (5,)
  want = [c[0, -1], 2, c[2, 2], c[3, -1], c[4, -1]]      # full row; the EOS; the last token before padding
  assert out.scores.tolist() == [float(x) for x in want]
  whole = inference_worker.InferenceWorker({"reward": Scorer()})
  assert whole.score(request=datatypes.ScoreRequest(prompt_tokens=p, completion_tokens=c)).scores.tolist() == out.scores.tolist()

  class PerSequence(torch.nn.Module):                    # a head that already gives one number per row
    def __init__(self):
      super().__init__()
      self.w = torch.nn.Parameter(torch.ones(1))

    def forward(self, ids, positions, cache, mask):
      return ids.float().sum(-1) * self.w, None
  seq = inference_worker.InferenceWorker({"reward": PerSequence()}).score(
      request=datatypes.ScoreRequest(prompt_tokens=p, completion_tokens=c))
  assert seq.scores.shape == (5,)


def test_replies_survive_the_wire():
  from tunix_b200.experimental.common import rpc_utils
  resp = datatypes.LogprobsResponse(request_id="r", per_token_logps=np.arange(6, dtype=np.float32).reshape(2, 3), model_version=4)
  back = rpc_utils.decode(rpc_utils.encode(resp)) if hasattr(rpc_utils, "encode") else resp
  assert back.request_id == "r" and back.model_version == 4 and np.array_equal(back.per_token_logps, resp.per_token_logps)


# ---- trainer worker ------------------------------------------------------------------------------
class FakeTrainer:
  def __init__(self):
    self.calls, self.policy_version, self.fail = [], 0, False

  def fwd_bwd(self, payload, **kw):
    if self.fail:
      raise RuntimeError("nan in loss")
    self.calls.append(("fwd_bwd", payload, kw))
    return {"loss": 0.5}

  def update(self, **kw):
    self.policy_version += 1
    self.calls.append(("update",))
    return self.policy_version

  def eval_step(self, payload, **kw):
    self.calls.append(("eval", payload))
    return {"eval_loss": 0.25}

  def save_checkpoint(self, force=False):
    return force

  def compile(self, dummy):
    self.calls.append(("compile", dummy))

  def close(self):
    self.calls.append(("close",))

  def state_for_weight_sync(self):
    return {"w": torch.ones(2, 2)}


def test_trainer_worker_replies_carry_state_and_version_and_failures_stick():
  t = FakeTrainer()
  w = trainer_worker.TrainerWorker(lambda: t, worker_id="t0")
  assert w.state == S.PENDING
  r = w.train_step({"x": 1}, skip_jit=True)              # initialises on the way; the compiler switch is dropped
  assert w.state == S.READY and t.calls[0] == ("fwd_bwd", {"x": 1}, {})
  assert r.metadata["loss"] == 0.5 and r.metadata["train_steps"] == 1 and r.metadata["policy_version"] == 1
  assert r.metadata["worker_id"] == "t0" and r.metadata["state"] == "READY"
  only_grads = w.train_step({"x": 2}, apply_optimizer=False)
  assert "train_steps" not in only_grads.metadata and w.policy_version == 1
  assert w.eval_step({"x": 3}).metadata["eval_loss"] == 0.25
  assert w.run_eval(None).metadata["eval_batches"] == 0 and w.run_eval([1, 2, 3]).metadata["batches"] == 3
  assert w.save_checkpoint(force=True).metadata["saved"] is True
  assert w.compile("dummy").metadata["compiled"] and ("compile", "dummy") in t.calls and w.state == S.READY
  assert w.start().metadata["started"] and w.initialize().metadata["already_ready"]
  assert w.heartbeat().policy_version == 1 and w.info().resources["trainer"] == "FakeTrainer"
  t.fail = True
  with pytest.raises(RuntimeError, match="nan in loss"):
    w.fwd_bwd({"x": 4})
  assert w.state == S.ERROR and w.heartbeat().last_error == "nan in loss"
  with pytest.raises(RuntimeError, match="not ready: ERROR"):
    w.fwd_bwd({"x": 5})
  assert w.stop().metadata["stopped"] and ("close",) in t.calls and w.state == S.STOPPED
  assert w.stop().metadata["already_stopped"]


def test_trainer_worker_is_syncing_between_prepare_and_release():
  t = FakeTrainer()
  attached = {}

  class Handler:
    def attach(self, unit, tensors):
      attached[unit.job_replica_id] = tensors
  w = trainer_worker.TrainerWorker(lambda: t, worker_id="t0", handler=Handler(), rank=2)
  w.initialize()
  meta = asyncio.run(w.prepare_weight_sync("req"))
  assert w.state == S.SYNCING and len(meta) == 1 and list(attached) == ["t0"] and w.work_unit.data_replica_idx == 2
  with pytest.raises(RuntimeError, match="not ready: SYNCING"):
    w.fwd_bwd({"x": 1})                                    # weights must not move under the transfer
  assert w.state == S.SYNCING                              # the refusal is not an error of the worker
  assert asyncio.run(w.release_weight_sync("req")) is None and w.state == S.READY
  w.fwd_bwd({"x": 1})


def test_trainer_hooks_are_used_when_the_trainer_stages_its_own_weights():
  class Staging(FakeTrainer):
    def prepare_weight_sync(self, sync_request=None, **kw):
      self.calls.append(("prepare", sync_request))
      return [{"unit": "trainer0"}]

    async def release_weight_sync(self, sync_request=None, **kw):
      self.calls.append(("release", sync_request))
      return "released"
  t = Staging()
  w = trainer_worker.TrainerWorker(lambda: t, worker_id="t0")
  req = object()
  assert asyncio.run(w.prepare_weight_sync(req)) == [{"unit": "trainer0"}] and w.state == S.SYNCING
  assert asyncio.run(w.release_weight_sync(req)) == "released" and w.state == S.READY
  assert t.calls == [("prepare", req), ("release", req)]

  class Broken(FakeTrainer):
    def state_for_weight_sync(self):
      raise RuntimeError("boom")
  bad = trainer_worker.TrainerWorker(lambda: Broken(), worker_id="t1")
  with pytest.raises(RuntimeError, match="boom"):
    asyncio.run(bad.prepare_weight_sync())
  assert bad.state == S.ERROR and bad.heartbeat().last_error == "boom"


# ---- rollout worker ------------------------------------------------------------------------------
class FakeManager:
  def __init__(self):
    self.calls, self.status = [], {"phase": "idle"}
    self.sampler = type("S", (), {"policy_version": 3, "initialize": lambda self: None})()

  def _note(self, phase, req):
    cfg = getattr(req, "extra_config", {}) or {}
    self.status = {"phase": phase, **cfg}

  async def bind_weight_sync(self, **kw):
    self.calls.append("bind")

  async def get_weight_sync_metadata(self, **kw):
    self.calls.append("metadata")
    return [{"unit": "u0"}]

  async def get_weight_sync_status(self, **kw):
    return dict(self.status)

  async def pre_weight_sync(self, req=None, **kw):
    self.calls.append("pre"); self._note("prepared", req)

  async def weight_sync(self, req=None, **kw):
    self.calls.append("sync"); self._note("h2d_done", req)

  async def post_weight_sync(self, req=None, **kw):
    self.calls.append("post"); self._note("committed", req)

  async def abort_weight_sync(self, req=None, **kw):
    self.calls.append("abort"); self._note("aborted", req)

  async def generate(self, reqs):
    self.calls.append(("generate", len(reqs)))
    if any(r.prompt == "explode" for r in reqs):
      raise RuntimeError("sampler died")
    return [datatypes.RolloutResponse(request_id=r.request_id, prompt_id=r.prompt_id, status="ok") for r in reqs]


class Req:
  def __init__(self, req_id, uuid):
    self.extra_config = {"req_id": req_id, "uuid": uuid}


def _rollout_worker():
  m = FakeManager()
  w = rollout_worker.RolloutWorker(lambda: m, worker_id="w0")
  w.initialize()
  return w, m


def test_rollout_worker_phases_move_the_state_and_reach_the_manager_in_order():
  async def go():
    w, m = _rollout_worker()
    req = Req("r1", 1)
    await w.bind_weight_sync()
    assert await w.get_weight_sync_metadata() == [{"unit": "u0"}]
    await w.pre_weight_sync(req)
    assert w.state == S.SYNCING
    assert await w.get_weight_sync_status() == {"phase": "prepared", "req_id": "r1", "uuid": 1}
    await w.weight_sync(req)
    await w.post_weight_sync(req)
    assert w.state == S.READY and m.calls == ["bind", "metadata", "pre", "sync", "post"]
    await w.pre_weight_sync(Req("r2", 2))
    await w.abort_weight_sync(Req("r2", 2))
    assert w.state == S.READY and (await w.get_weight_sync_status())["phase"] == "aborted"
  asyncio.run(go())


def test_rollout_worker_generate_counts_inflight_and_keeps_the_last_error():
  async def go():
    w, m = _rollout_worker()
    seen = []
    inner = m.generate

    async def watched(reqs):
      seen.append(w.heartbeat().inflight)
      return await inner(reqs)
    m.generate = watched
    out = await w.generate(prompts=["a", "b"], temperature=0.5)
    assert [r.request_id for r in out] == ["w0_1", "w0_2"] and seen == [2] and w.heartbeat().inflight == 0
    assert w.heartbeat().policy_version == 3
    with pytest.raises(RuntimeError, match="sampler died"):
      await w.generate(prompts=["explode"])
    assert w.heartbeat().last_error == "sampler died" and w.heartbeat().inflight == 0
    w.stop()
    with pytest.raises(RuntimeError, match="not ready: STOPPED"):
      await w.generate(prompts=["a"])
  asyncio.run(go())
  fresh = rollout_worker.RolloutWorker(lambda: FakeManager())
  with pytest.raises(RuntimeError, match="Cannot start RolloutWorker from PENDING"):
    fresh.start()


# ---- admission gate ------------------------------------------------------------------------------
def test_the_gate_admits_while_ready_numbers_epochs_and_cancels_on_stop():
  async def go():
    tc = traffic_controller.TrafficController()
    assert tc.state == S.READY and tc.is_admission_open() and tc.epoch == 0 and tc.get_active_tasks() == []
    hold = asyncio.Event()

    async def work():
      await hold.wait()
      return "done"
    first = asyncio.create_task(work())
    assert tc.try_admit(first) and tc.get_active_tasks() == [first]
    tc.transition_to_syncing()
    tc.transition_to_syncing()                             # idempotent
    refused = asyncio.create_task(work())
    assert not tc.try_admit(refused)
    await asyncio.sleep(0)
    assert refused.cancelled() or refused.cancelling()
    waiter = asyncio.create_task(tc.wait_for_admission())
    await asyncio.sleep(0.01)
    assert not waiter.done()
    await tc.drain(0.05)                                   # the old task is still running: the drain times out
    assert not first.done()
    hold.set()
    await tc.drain(1.0)
    assert first.done() and tc.get_active_tasks() == []
    assert tc.reopen() and tc.epoch == 1
    await asyncio.wait_for(waiter, 1.0)
    assert tc.reopen() and tc.epoch == 1                   # reopening an open gate starts no new epoch
    hold.clear()
    tracked = asyncio.create_task(work())
    tc.track(tracked)
    doomed = tc.stop_and_cancel_all()
    await asyncio.sleep(0)
    assert doomed == [tracked] and tc.state == S.STOPPED and not tc.reopen()
    with pytest.raises(asyncio.CancelledError):
      await tracked
    with pytest.raises(RuntimeError, match="Cannot transition to SYNCING from STOPPED"):
      tc.transition_to_syncing()
    assert issubclass(traffic_controller.AdmissionClosedError, RuntimeError)
  asyncio.run(go())


def test_the_gate_can_be_driven_from_another_thread():
  import threading

  async def go():
    tc = traffic_controller.TrafficController()
    tc.transition_to_syncing()
    waiter = asyncio.create_task(tc.wait_for_admission())
    await asyncio.sleep(0.01)
    threading.Thread(target=tc.reopen).start()             # e.g. the RPC thread that finishes a weight sync
    await asyncio.wait_for(waiter, 2.0)
    t = asyncio.create_task(asyncio.sleep(10))
    tc.try_admit(t)
    th = threading.Thread(target=tc.stop_and_cancel_all)
    th.start(); th.join()
    with pytest.raises(asyncio.CancelledError):
      await asyncio.wait_for(t, 2.0)
  asyncio.run(go())
