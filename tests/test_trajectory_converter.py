"""Action shapes -> tool calls, and the episode <-> stored-trajectory round trip."""
import dataclasses
import types

import numpy as np
import pytest

from tunix_b200.experimental.trajectory import action_converter as ac, converter, trajectory as tl
from tunix_b200.rl.agentic.agents import agent_types


def _sig(calls):
  return [(c.tool_call_id, c.function_name, c.arguments) for c in calls or []]


def test_action_shapes():
  openai = {"id": "x1", "type": "function", "function": {"name": "search", "arguments": '{"q": "b200"}'}}
  assert _sig(ac.extract_tool_calls(agent_types.Action(action=[openai]))) == [("x1", "search", {"q": "b200"})]
  anthropic = {"type": "tool_use", "id": "tu", "name": "calc", "input": {"e": "1+1"}}
  assert _sig(ac.extract_tool_calls(anthropic)) == [("tu", "calc", {"e": "1+1"})]
  assert _sig(ac.extract_tool_calls({"name": "move", "dx": 1, "dy": 2})) == [("call_1", "move", {"dx": 1, "dy": 2})]
  assert _sig(ac.extract_tool_calls({"direction": "up"})) == [("call_1", "action", {"direction": "up"})]
  assert ac.extract_tool_calls({"id": "only"}) is None
  for not_a_call in (None, 3, 2.5, True, np.int64(4), np.zeros(3), "", [], {}, "just some prose"):
    assert ac.extract_tool_calls(not_a_call) is None

  @dataclasses.dataclass
  class Call:
    tool_name: str
    params: dict

  nested = agent_types.Action(action=agent_types.Action(action=[Call("a", {"k": 1}), Call("b", {})]))
  assert _sig(ac.extract_tool_calls(nested)) == [("call_1", "a", {"k": 1}), ("call_2", "b", {})]
  slotted = types.SimpleNamespace(function_name="f", args='```json\n{"z": 1}\n```', call_id="c9")
  assert _sig(ac.extract_tool_calls(slotted)) == [("c9", "f", {"z": 1})]
  ready = tl.ToolCall(tool_call_id="t", function_name="n", arguments={})
  assert ac.extract_tool_calls(ready) == [ready]


def test_action_text_formats():
  text = ('I will look.\n<tool_call>\n{"name": "search", "arguments": {"q": "x"}}\n</tool_call>\n'
          '<tool_call><name>open</name><arguments>{"url": "u"}</arguments></tool_call>')
  assert _sig(ac.extract_tool_calls(text)) == [("call_1", "search", {"q": "x"}), ("call_2", "open", {"url": "u"})]
  xml = '<function=grep>\n<parameter=pattern>foo</parameter>\n<parameter=path>"."</parameter>\n</function>'
  assert _sig(ac.extract_tool_calls(xml)) == [("call_1", "grep", {"pattern": "foo", "path": '"."'})]
  invoke = '<invoke name="run">ls -l</invoke><invoke name="json">{"a": 1}</invoke><invoke name="none"></invoke>'
  assert _sig(ac.extract_tool_calls(invoke)) == [("call_1", "run", {"input": "ls -l"}), ("call_2", "json", {"a": 1}),
                                                 ("call_3", "none", {})]
  fenced = '```json\n[{"name": "a", "args": {"x": 1}}, {"function": {"name": "b"}}]\n```'
  assert _sig(ac.extract_tool_calls(fenced)) == [("call_1", "a", {"x": 1}), ("call_2", "b", {})]
  assert ac.extract_tool_calls("{not json") is None


def _episode():
  s0 = agent_types.Step(model_response="call search", thought="hmm",
                        action=agent_types.Action(action=[{"id": "c", "function": {"name": "search", "arguments": {"q": 1}}}]),
                        observation={"tool_outputs": {"c": "found"}}, reward=0.0, done=False, mc_return=0.5,
                        assistant_tokens=np.array([5, 6, 7]), assistant_masks=np.array([1, 1, 1]),
                        env_tokens=np.array([9, 9]), env_masks=np.array([0, 0]), logprobs=np.array([-0.1, -0.2, -0.3]),
                        info={"turn": 0})
  s1 = agent_types.Step(model_response="42", action=agent_types.Action(action="42"), observation=None, reward=1.0,
                        done=True, assistant_tokens=np.array([8]), assistant_masks=np.array([1]),
                        logprobs=np.array([-0.5]))
  return agent_types.Trajectory(task={"prompts": ["what is it?"]}, steps=[s0, s1], reward=1.0,
                                status=agent_types.TrajectoryStatus.SUCCEEDED, env_time={"t": 0.1})


def test_episode_round_trip_through_the_stored_schema():
  ep = _episode()
  req = types.SimpleNamespace(prompt_id="p7", group_offset_id="2", generation_kwargs={"temperature": 0.9},
                              metadata={"group_id": "g"})
  stored = converter.from_tunix_trajectory(ep, "traj-1", request=req, agent=types.SimpleNamespace(name="a", version="2"),
                                           target_policy_versions=[3])
  assert [s.step_id for s in stored.steps] == [0, 1, 2, 3, 4]
  assert [s.source.value for s in stored.steps] == ["user", "agent", "system", "agent", "system"]
  assert stored.steps[1].tool_calls[0].function_name == "search" and stored.steps[1].metrics.completion_tokens == 3
  assert stored.prompt_id == "p7" and stored.total_reward == 1.0 and stored.status == "SUCCEEDED"
  back = converter.to_tunix_trajectory(tl.TunixTrajectory.from_json_dict(stored.to_json_dict()))
  assert back.task == ep.task and back.reward == 1.0 and back.status == agent_types.TrajectoryStatus.SUCCEEDED
  assert len(back.steps) == 2
  for a, b in zip(ep.steps, back.steps):
    assert a.model_response == b.model_response and a.thought == b.thought and a.reward == b.reward and a.done == b.done
    assert a.action.action == b.action.action
    np.testing.assert_array_equal(a.assistant_tokens, b.assistant_tokens)
    np.testing.assert_allclose(a.logprobs, b.logprobs)
  assert back.steps[0].info == {"turn": 0} and back.steps[0].mc_return == 0.5
  assert back.steps[0].observation == str(ep.steps[0].observation)


def test_incremental_writer_and_loose_records():
  w = converter.EpisodeWriter()
  ep = _episode()
  steps = w.task(ep.task) + w.turn(ep.steps[0])
  assert [s.step_id for s in steps] == [0, 1, 2] and w.turns == 1
  with pytest.raises(ValueError, match="must match"):
    converter.create_agent_step(agent_types.Step(assistant_tokens=np.array([1, 2]), logprobs=np.array([0.1])), 0)
  assert converter.create_task_step({"prompts": []}) is None and converter.create_task_step("") is None
  # an agent step directly followed by another agent step, then a lone environment step
  a1 = tl.TunixAgentStep(step_id=0, source=tl.Source.AGENT, message="one", tool_calls=[
      tl.ToolCall(tool_call_id="i", function_name="f", arguments={"x": 1})])
  a2 = tl.TunixAgentStep(step_id=1, source=tl.Source.AGENT, message="two")
  e3 = tl.TunixEnvStep(step_id=2, source=tl.Source.SYSTEM, message="obs", reward=0.25, done=True)
  e4 = tl.TunixEnvStep(step_id=3, source=tl.Source.SYSTEM, message="late")
  loose = tl.TunixTrajectory(agent=tl.Agent(name="x"), steps=[a1, a2, e3, e4])
  turns = converter.to_tunix_trajectory(loose).steps
  assert [(t.model_response, t.observation, t.reward) for t in turns] == [("one", None, 0.0), ("two", "obs", 0.25),
                                                                          ("", "late", 0.0)]
  assert turns[0].action.action == {"id": "i", "name": "f", "arguments": {"x": 1}}
