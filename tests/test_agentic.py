"""Agentic building blocks on CPU: tools, parsers, environments, engine, orchestrator, lock."""
import asyncio
import threading
import time
from types import SimpleNamespace

import numpy as np
import pytest

from tunix_b200.rl.agentic import utils as autils
from tunix_b200.rl.agentic.agents import agent_types, model_agent, tool_agent
from tunix_b200.rl.agentic.environments import task_environment, tool_environment
from tunix_b200.rl.agentic.parser.chat_template_parser import parser as ctp
from tunix_b200.rl.agentic.parser.tool_parser import tool_parser_registry
from tunix_b200.rl.agentic.pipeline.rollout_orchestrator import RolloutOrchestrator
from tunix_b200.rl.agentic.queue_manager.group_queue_manager import GroupQueueManager
from tunix_b200.rl.agentic.rewards import reward
from tunix_b200.rl.agentic.tools import base_tool, calculator_tool, tool_manager
from tunix_b200.rl.agentic.trajectory.trajectory_collect_engine import TrajectoryCollectEngine


class CharTok:
  bos_token, eos_token = "<s>", "</s>"
  def encode(self, s, add_special_tokens=False): return [ord(c) % 251 + 3 for c in s]
  def decode(self, ids): return "".join(chr(i) for i in ids)
  def dedup_bos_ids(self, ids): return ids
  def bos_id(self): return 1
  def eos_id(self): return 2
  def pad_id(self): return 0


def out(text, n=None):
  toks = np.arange(n if n is not None else len(text)) + 5
  return SimpleNamespace(text=[text], tokens=[toks], logprobs=[-0.5 * np.ones(len(toks), np.float32)],
                         left_padded_prompt_tokens=None)


def test_tools_and_parsers():
  tm = tool_manager.ToolManager({"calculator": calculator_tool.CalculatorTool})
  assert str(tm.run("calculator", a=6, b=3, op="/")) == "2.0"
  assert "Division by zero" in str(tm.run("calculator", a=1, b=0, op="/"))
  assert "not registered" in str(tm.run("nope"))
  calc = tm.get_tools()[0]
  with pytest.raises(AttributeError):
    calc.name = "x"
  res = tm.execute_calls([base_tool.ToolCall("calculator", {"a": 2, "b": 5, "op": "*"}),
                          base_tool.ToolCall("calculator", {"a": 2, "b": 5, "op": "+"})])
  assert sorted(res.values()) == ["10", "7"]
  qp = tool_parser_registry.get_tool_parser("qwen")()
  calls = qp.parse('think <tool_call>{"name": "calculator", "arguments": {"a": 1, "b": 2, "op": "+"}}</tool_call>'
                   ' <tool_call>{broken</tool_call>')
  assert len(calls) == 1 and calls[0].name == "calculator" and calls[0].arguments["op"] == "+"
  assert "<tools>" in qp.get_tool_prompt([calc]) and '"calculator"' in qp.get_tool_prompt([calc])
  with pytest.raises(ValueError):
    tool_parser_registry.get_tool_parser("zzz")
  with pytest.raises(TypeError):
    tool_manager.ToolManager({"abstract": base_tool.BaseTool})


def test_chat_template_parsers_incremental_equals_whole():
  tok = CharTok()
  msgs = [{"role": "system", "content": "sys"}, {"role": "user", "content": "hi <|im_end|>there"},
          {"role": "assistant", "content": "yo"}, {"role": "tool", "content": "42"}]
  for cls in (ctp.QwenChatTemplateParser, ctp.LlamaChatTemplateParser, ctp.Gemma4ChatTemplateParser):
    p = cls(tok)
    whole = p.parse(msgs, add_generation_prompt=True, is_first_msg=True)
    pieces = p.parse(msgs[:1], is_first_msg=True) + "".join(p.parse([m]) for m in msgs[1:-1]) + \
        p.parse(msgs[-1:], add_generation_prompt=True)
    assert whole == pieces, cls.__name__
  q = ctp.QwenChatTemplateParser(tok)
  s = q.parse(msgs[1:2], is_first_msg=True)
  assert s.startswith("<|im_start|>system\nYou are Qwen") and "hi there" in s and s.count("<|im_end|>") == 2
  g = ctp.GemmaChatTemplateParser(tok)
  assert g.parse(msgs[:2]) == "<start_of_turn>user\nsys\nhi <|im_end|>there<end_of_turn>\n"
  assert "<think>\n\n</think>" in ctp.QwenChatTemplateParser(tok, enable_thinking=False).generation_prompt


def test_rewards_registry():
  assert reward.get_reward_fn("exact_match")({"ground_truth": " 4 "}, "4").reward == 1.0
  assert reward.calculate_reward({"question": "2 * (3 + 4) = ?"}, "The answer is 14.").reward == 1.0
  assert reward.calculate_reward({"question": "__import__('os')"}, "1").reward == 0.0
  combo = reward.combine_rewards({"exact_match": 0.5, "is_two": 2.0})
  assert combo({"ground_truth": "2"}, "2").reward == 2.5
  with pytest.raises(ValueError):
    reward.register("dummy")(lambda t, a: None)


def test_rollout_sync_lock_prefers_weight_sync():
  lock = autils.RolloutSyncLock()
  events = []
  lock.acquire_rollout()
  def sync():
    lock.acquire_weight_sync(); events.append("sync"); time.sleep(0.05); lock.release_weight_sync()
  def late_rollout():
    lock.acquire_rollout(); events.append("rollout2"); lock.release_rollout()
  t1 = threading.Thread(target=sync); t1.start(); time.sleep(0.05)
  t2 = threading.Thread(target=late_rollout); t2.start(); time.sleep(0.05)
  assert events == []            # sync waits for the running rollout, the new rollout waits for the sync
  lock.release_rollout()
  t1.join(2); t2.join(2)
  assert events == ["sync", "rollout2"]


def test_group_queue_manager_groups_filters_and_propagates():
  async def run():
    m = GroupQueueManager(group_size=2, key_fn=lambda x: x[0], filter_fn=lambda g: [x for x in g if x[1] >= 0])
    for item in [("a", 1), ("b", 2), ("a", -1), ("b", 3), ("c", 1)]:
      await m.put(item)
    b = await m.get_batch(3)
    assert b == [("a", 1), ("b", 2), ("b", 3)]
    assert await m.get_filtered_groups() == [[("a", -1)]]
    await m.put_exception(RuntimeError("boom"))
    with pytest.raises(RuntimeError):
      await m.get_batch(1)
    with pytest.raises(ValueError):
      GroupQueueManager()
  asyncio.run(run())


def test_single_turn_episode_token_mode():
  tok = CharTok()
  env = task_environment.TaskEnvironment({"question": "1 + 1 = ?"}, reward_fn=lambda task, action: float(action == "2"),
                                         group_id=7, pair_index=0)
  agent = model_agent.ModelAgent("be brief")
  eng = TrajectoryCollectEngine(agent, env, model_call=lambda msgs, env, **kw: out("2"), tokenizer=tok,
                                chat_parser=ctp.QwenChatTemplateParser(tok))
  res = asyncio.run(eng.collect("Token"))
  assert res["status"] == "SUCCEEDED" and res["trajectory_reward"] == 1.0 and res["group_id"] == 7
  assert res["conversation_masks"].tolist() == [1] and len(res["old_logprobs"]) == 1
  assert len(res["prompt_tokens"]) > 10


def test_tool_episode_multi_turn_and_limits():
  tok = CharTok()
  replies = iter(['<tool_call>{"name": "calculator", "arguments": {"a": 20, "b": 22, "op": "+"}}</tool_call>', "42"])
  env = tool_environment.ToolEnvironment({"question": "20+22?"}, tool_map={"calculator": calculator_tool.CalculatorTool},
                                         reward_fn=lambda task, action: float(action.strip() == "42"), max_steps=4,
                                         pair_index=0, group_id=0)
  agent = tool_agent.ToolAgent("solve", tool_map={"calculator": calculator_tool.CalculatorTool})
  eng = TrajectoryCollectEngine(agent, env, model_call=lambda m, e, **kw: out(next(replies)), gamma=0.5, tokenizer=tok,
                                chat_parser=ctp.QwenChatTemplateParser(tok))
  traj = asyncio.run(eng.collect("Trajectory"))
  assert traj.status == agent_types.TrajectoryStatus.SUCCEEDED and len(traj.steps) == 2
  assert traj.reward == 1.0 and traj.steps[0].mc_return == 0.5 and traj.steps[1].mc_return == 1.0
  assert "Tool returned result: 42" in agent.chat_completions[-2]["content"]
  assert traj.steps[0].env_tokens is not None and set(traj.steps[0].env_masks.tolist()) == {0}
  # max steps reached -> masks zeroed under the overlong filter
  env2 = tool_environment.ToolEnvironment({"question": "?"}, tool_map={"calculator": calculator_tool.CalculatorTool},
                                          reward_fn=lambda task, action: 1.0, max_steps=2, pair_index=0, group_id=0)
  call = '<tool_call>{"name": "calculator", "arguments": {"a": 1, "b": 1, "op": "+"}}</tool_call>'
  agent2 = tool_agent.ToolAgent("solve", tool_map={"calculator": calculator_tool.CalculatorTool})
  eng2 = TrajectoryCollectEngine(agent2, env2, model_call=lambda m, e, **kw: out(call), tokenizer=tok,
                                 chat_parser=ctp.QwenChatTemplateParser(tok), overlong_filter=True)
  eng2.max_steps = 1        # the engine's own turn limit, below the environment's
  res = asyncio.run(eng2.collect("Token"))
  assert res["status"] == "MAX_STEPS_REACHED" and res["conversation_masks"].sum() == 0
  # response-token budget
  eng3 = TrajectoryCollectEngine(tool_agent.ToolAgent("s", tool_map={"calculator": calculator_tool.CalculatorTool}),
                                 tool_environment.ToolEnvironment({"question": "?"}, tool_map={"calculator": calculator_tool.CalculatorTool}, max_steps=5, pair_index=0),
                                 model_call=lambda m, e, **kw: out(call, 30), tokenizer=tok, max_response_length=40,
                                 chat_parser=ctp.QwenChatTemplateParser(tok))
  assert asyncio.run(eng3.collect("Trajectory")).status == agent_types.TrajectoryStatus.MAX_CONTEXT_LIMIT_REACHED


def test_env_timeout_status():
  class SlowEnv(task_environment.TaskEnvironment):
    def step(self, action):
      time.sleep(0.5)
      return super().step(action)
  eng = TrajectoryCollectEngine(model_agent.ModelAgent(""), SlowEnv({"question": "q"}, reward_fn=lambda **k: 1.0, pair_index=0),
                                model_call=lambda m, e, **kw: out("x"), timeout=0.1)
  traj = asyncio.run(eng.collect("Trajectory"))
  assert traj.status == agent_types.TrajectoryStatus.ENV_TIMEOUT and traj.reward == 0.0


def test_orchestrator_groups_and_propagates_failure():
  def pairs(n_groups, g, fail_at=None):
    for gid in range(n_groups):
      for j in range(g):
        idx = gid * g + j
        def rf(task, action, idx=idx):
          if fail_at == idx:
            raise RuntimeError("reward exploded")
          return float(idx)
        yield model_agent.ModelAgent(""), task_environment.TaskEnvironment({"question": str(gid)}, reward_fn=rf,
                                                                           group_id=gid, pair_index=idx)

  async def run(fail_at=None):
    orch = RolloutOrchestrator(rollout_sync_lock=autils.RolloutSyncLock(), max_concurrency=3,
                               engine_kwargs={"model_call": lambda m, e, **kw: out("a")})
    prod = asyncio.create_task(orch.run_producers_from_stream(
        pairs(3, 2, fail_at), group_size=2, group_key_fn=lambda i, env, traj: env.extra_kwargs["group_id"],
        collect_mode="Trajectory"))
    got = []
    async for batch in orch.yield_batches(2):
      got.append(batch)
    await asyncio.gather(prod, return_exceptions=True)
    return got

  batches = asyncio.run(run())
  assert len(batches) == 3
  for b in batches:
    assert len(b) == 2 and b[0].group_id == b[1].group_id
  assert sorted(i.pair_index for b in batches for i in b) == list(range(6))
  with pytest.raises(RuntimeError, match="reward exploded"):
    asyncio.run(run(fail_at=3))


def test_frozenlake_environment_and_oracle():
  from tunix_b200.examples import frozenlake
  from tunix_b200.examples.frozenlake import env as fl
  for seed in range(5):
    e = frozenlake.FrozenLakeEnv({"size": 5, "p_hole": 0.3, "seed": seed}, max_steps=20)
    obs, _ = e.reset()
    assert "P" in obs["question"] and "G" in obs["question"]
    path = fl.shortest_path_moves(e)
    assert path
    reward = done = None
    for mv in path:
      obs, reward, done, info = e.step(f"I think ```{mv.capitalize()}```")
      assert info["valid"]
    assert done and reward == 1.0
  e = frozenlake.FrozenLakeEnv.from_dict({"size": 3, "seed": 1, "max_steps": 2})
  e.reset()
  _, r, d, info = e.step("no idea")
  assert not info["valid"] and r == 0.0 and not d
  _, r, d, _ = e.step("left")
  assert d                                  # step budget reached
  assert fl.parse_move("first Up, then ```Down```") == "down"
  agent = frozenlake.FrozenLakeAgent()
  assert "frozen lake" in agent.system_prompt


def test_function_tool_schema_freeze_and_ordered_parallel_execution():
  from tunix_b200.rl.agentic.tools import base_tool, tool_manager

  def add(a: int, b: int = 1):
    """Adds two integers."""
    return {"sum": a + b}

  tool = base_tool.FunctionTool(add)
  fn = tool.get_json_schema()["function"]
  assert fn["name"] == "add" and fn["description"] == "Adds two integers."
  assert fn["parameters"]["required"] == ["a"] and fn["parameters"]["properties"]["b"]["type"] == "integer"
  with pytest.raises(AttributeError):
    tool.name = "other"                      # frozen once the outermost constructor returned
  mgr = tool_manager.ToolManager({})
  mgr.register_mcp_tool(tool)
  calls = []
  for i in range(5):
    c = base_tool.ToolCall(name="add", arguments={"a": i})
    c.id = f"call{i}"
    calls.append(c)
  bad = base_tool.ToolCall(name="nope", arguments={})
  bad.id = "bad"
  out = mgr.execute_calls(calls + [bad], parallel=True)
  assert list(out) == [f"call{i}" for i in range(5)] + ["bad"]
  assert out["call3"] == '{"sum": 4}' and "not registered" in out["bad"]


def test_frozen_after_init_mixin():
  from tunix_b200.utils.immutable import FrozenAfterInit

  class Base(FrozenAfterInit):
    def __init__(self, a):
      self.a = a
      super().__init__()

  class Child(Base):
    def __init__(self, a, b):
      self.b = b                 # before and after the parent's constructor: both are still construction
      super().__init__(a)
      self.c = a + b

  class Plain(FrozenAfterInit):
    pass

  x = Child(1, 2)
  assert (x.a, x.b, x.c) == (1, 2, 3)
  for mutate in (lambda: setattr(x, "a", 5), lambda: delattr(x, "b"), lambda: setattr(Plain(), "z", 1),
                 lambda: setattr(Base(1), "a", 2)):
    with pytest.raises(AttributeError, match="immutable"):
      mutate()
  with x.thaw():
    x.a = 10
  assert x.a == 10
  with pytest.raises(AttributeError):
    x.a = 11
