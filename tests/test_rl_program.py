"""`StandardRLProgram` over a scripted engine: the four stages end to end, back-pressure by staleness, optimizer
cadence over micro-batches and groups, reference log-probs for KL, prompt ids, stage failures, cancellation, and the
synchronous entry point inside a running loop."""
import asyncio
import time

import numpy as np
import pytest

from tunix_b200.experimental.common import datatypes
from tunix_b200.experimental.orchestrator import algorithm_adapter, batch_assembly, rl_program
from tunix_b200.rl import common as rl_common


class ScriptedEngine:
  """Rollouts finish `latency` seconds after dispatch; everything the program asks is recorded."""

  def __init__(self, latency=0.0, fail=None):
    self.latency, self.fail = latency, fail or set()
    self.pending, self.dispatched, self.train_calls, self.syncs, self.ref_calls = [], [], [], 0, 0
    self.version = 0

  async def dispatch_rollouts(self, items, group_size, policy_version, **kw):
    if "dispatch" in self.fail:
      raise ConnectionError("rollout workers are gone")
    for item in items:
      self.dispatched.append((item["prompt_id"], policy_version, time.monotonic()))
      for k in range(group_size):
        traj = datatypes.TrajectoryItem(pair_index=k, group_id=item["prompt_id"], start_step=0,
                                        traj=datatypes.Trajectory(reward=float(k)),
                                        prompt_tokens=np.array([1, 2]), completion_tokens=np.array([3 + k, 4, 5]),
                                        policy_version=policy_version)
        self.pending.append((time.monotonic() + self.latency, traj))

  async def poll_rollouts(self, timeout_s=0.2):
    await asyncio.sleep(0.005)
    now = time.monotonic()
    ready = [t for due, t in self.pending if due <= now]
    self.pending = [(due, t) for due, t in self.pending if due > now]
    return ready

  async def train_step(self, batch, role, accumulate_gradients, apply_optimizer):
    if "train" in self.fail:
      raise FloatingPointError("loss is NaN")
    self.train_calls.append((type(batch).__name__, apply_optimizer, getattr(batch, "ref_per_token_logps", None) is not None))
    return {"loss": 0.5}

  async def per_token_logps(self, role, items):
    self.ref_calls += 1
    assert role == datatypes.Role.REFERENCE
    return np.zeros(np.asarray(items.completion_ids).shape, np.float32)

  async def sync_weights(self, role):
    self.syncs += 1
    self.version += 1
    return self.version


def program(group_size=2, mini=1, beta=0.0, batch=2, **kw):
  algo = algorithm_adapter.GRPOAdapter(group_size=group_size, mini_batch_size=mini, beta_kl=beta)
  assembler = batch_assembly.GRPOTrainExampleAssembler(batch_size=batch, max_prompt_length=4, max_response_length=4, pad_id=0)
  return rl_program.StandardRLProgram(algo, assembler=assembler, **kw)


def prompts(n):
  return [f"question {i}" for i in range(n)]


def test_four_stages_end_to_end():
  engine, prog = ScriptedEngine(), program()
  seen = []
  prog.on_step_begin, prog.on_step_end = (lambda s: seen.append(("begin", s))), (lambda s, r: seen.append(("end", s)))
  prog.run(engine, prompts(3), num_steps=3)
  assert [r.policy_version for r in prog.history] == [1, 2, 3] and prog.step == 3 and engine.syncs == 3
  first = prog.history[0]
  assert first.num_rollouts == 2 and first.num_microbatches == 1 and first.reward_mean == 0.5 and first.reward_std == 0.5
  assert first.train_result == {"loss": 0.5} and prog.last_step_result is prog.history[-1]
  assert seen[:2] == [("begin", 0), ("end", 0)] and len(seen) == 6
  assert [p for p, _, _ in engine.dispatched] == ["prompt_0", "prompt_1", "prompt_2"]
  assert not prog._is_running


def test_the_data_running_out_ends_training_and_syncs_can_be_skipped():
  engine, prog = ScriptedEngine(), program(sync_weights=False)
  prog.run(engine, prompts(2), num_steps=10)
  assert len(prog.history) == 2 and engine.syncs == 0 and prog.policy_version == 2     # versions still count steps
  with pytest.raises(ValueError, match="requires a dataset"):
    program().run(ScriptedEngine(), None, num_steps=1)
  with pytest.raises(ValueError, match="max_staleness must be non-negative"):
    program(max_staleness=-1)
  at_init = rl_program.StandardRLProgram(algorithm_adapter.GRPOAdapter(group_size=2, mini_batch_size=1, beta_kl=0.0),
                                         dataset=prompts(1), assembler=program().assembler)
  at_init.run(ScriptedEngine(), num_steps=1)
  assert len(at_init.history) == 1


@pytest.mark.parametrize("staleness, ahead", [(0, 1), (1, 2), (None, 6)])
def test_dispatch_runs_at_most_max_staleness_steps_ahead(staleness, ahead):
  """How many prompts are out before the first optimizer step has finished."""
  engine, prog = ScriptedEngine(latency=0.05), program(max_staleness=staleness)
  counts = []
  prog.on_step_end = lambda step, result: counts.append(len(engine.dispatched))
  prog.run(engine, prompts(6), num_steps=3)
  assert counts[0] == ahead
  if staleness is not None:
    assert all(c <= (i + 1) + staleness + 1 for i, c in enumerate(counts))
    versions = {p: v for p, v, _ in engine.dispatched}
    assert all(int(p.split("_")[1]) - v <= staleness for p, v in versions.items())     # never more than that stale


def test_optimizer_applies_once_per_step_on_the_very_last_micro_batch():
  engine, prog = ScriptedEngine(), program(group_size=3, mini=2, batch=2)        # 3 rollouts -> 2 micro-batches per group
  prog.run(engine, prompts(4), num_steps=2)
  applied = [a for _, a, _ in engine.train_calls]
  assert applied == [False, False, False, True] * 2
  assert [r.num_microbatches for r in prog.history] == [4, 4] and [r.num_rollouts for r in prog.history] == [6, 6]
  assert engine.ref_calls == 0


def test_reference_logprobs_are_fetched_per_micro_batch_when_the_loss_has_a_kl_term():
  engine, prog = ScriptedEngine(), program(beta=0.04)
  prog.run(engine, prompts(2), num_steps=2)
  assert engine.ref_calls == 2 and all(has_ref for _, _, has_ref in engine.train_calls)
  packed = rl_program.StandardRLProgram(algorithm_adapter.GRPOAdapter(group_size=2, mini_batch_size=1, beta_kl=0.04),
                                        assembler=batch_assembly.SequencePackedBatchAssembler(16))
  with pytest.raises(TypeError, match="Reference KL requires an assembler that returns rl_common.TrainExample"):
    packed.run(ScriptedEngine(), prompts(1), num_steps=1)


def test_prompt_ids_are_kept_or_invented():
  assert rl_program._as_prompt_item("text", 3) == {"prompt": "text", "prompt_id": "prompt_3"}
  assert rl_program._as_prompt_item({"prompt": "p"}, 1) == {"prompt_id": "prompt_1", "prompt": "p"}
  assert rl_program._as_prompt_item({"prompt": "p", "prompt_id": "mine"}, 1)["prompt_id"] == "mine"
  class Item:
    prompt_id = "object"
  it = Item()
  assert rl_program._as_prompt_item(it, 0) is it


@pytest.mark.parametrize("stage, error", [("dispatch", ConnectionError), ("train", FloatingPointError)])
def test_a_failing_stage_ends_the_program_with_its_exception(stage, error):
  engine, prog = ScriptedEngine(fail={stage}), program()
  with pytest.raises(error):
    prog.run(engine, prompts(3), num_steps=3)
  assert not prog._is_running


def test_a_failing_reward_function_surfaces_too():
  def broken(item):
    raise KeyError("no answer field")
  prog = program(reward_fns=[broken])
  with pytest.raises(KeyError, match="no answer field"):
    prog.run(ScriptedEngine(), prompts(2), num_steps=1)


def test_external_cancellation_stops_all_stages():
  engine, prog = ScriptedEngine(latency=10.0), program()              # rollouts never arrive

  async def scenario():
    task = asyncio.create_task(prog.run_async(engine, prompts(2), num_steps=1))
    await asyncio.sleep(0.1)
    before = len(asyncio.all_tasks())
    task.cancel()
    with pytest.raises(asyncio.CancelledError):
      await task
    await asyncio.sleep(0.05)
    return before, len(asyncio.all_tasks())
  before, after = asyncio.run(scenario())
  assert before >= 5 and after == 1 and not prog._is_running          # only the test's own task is left


def test_the_synchronous_entry_point_works_inside_a_running_loop():
  engine, prog = ScriptedEngine(), program()

  async def caller():
    prog.run(engine, prompts(2), num_steps=2)                          # would be "asyncio.run() cannot be called..." otherwise
    return len(prog.history)
  assert asyncio.run(caller()) == 2
  failing = program()
  async def caller2():
    failing.run(ScriptedEngine(fail={"train"}), prompts(1), num_steps=1)
  with pytest.raises(FloatingPointError):
    asyncio.run(caller2())


def test_reward_functions_replace_environment_rewards_and_advantages_are_group_relative():
  seen = []
  engine = ScriptedEngine()
  real = engine.train_step

  async def spy(batch, **kw):
    seen.append(np.asarray(batch.advantages))
    return await real(batch, **kw)
  engine.train_step = spy
  prog = program(group_size=2, reward_fns=[lambda item: 10.0 * item.pair_index, lambda item: 1.0])
  prog.run(engine, prompts(1), num_steps=1)
  assert prog.history[0].reward_mean == 6.0                             # (1 + 11) / 2: both functions summed
  adv = seen[0].reshape(2, -1)[:, 0] if seen[0].ndim > 1 else seen[0]
  assert adv[0] == pytest.approx(-1.0, abs=1e-3) and adv[1] == pytest.approx(1.0, abs=1e-3)
