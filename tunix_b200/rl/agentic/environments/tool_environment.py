"""Multi-turn tool environment (tunix/rl/agentic/environments/tool_environment.py:36-248).

An action is normalised into a list of OpenAI-style tool calls or a plain string. A string, or a call to the
pseudo-tool `finish`, is the final answer: the episode ends and the answer is scored. Anything else is executed
through the `ToolManager` (calls of one turn run in parallel) and the outputs, keyed by call id, become the next
observation."""
from __future__ import annotations

import json
import logging
import uuid
from typing import Any, Dict, List, Optional, Type, Union

from ..agents import agent_types
from ..tools import base_tool, tool_manager
from . import base_environment

FINISH = "finish"


def _arguments(call: Dict[str, Any]) -> Any:
  """Arguments of a call as a dict where they parse as JSON, else the raw string."""
  raw = call["function"].get("arguments", {})
  if not isinstance(raw, str):
    return raw
  try:
    return json.loads(raw)
  except json.JSONDecodeError:
    return raw


def _calls_of(action: Any) -> Union[str, List[Dict[str, Any]]]:
  if isinstance(action, agent_types.Action):
    action = action.action
  if action is None:
    return []
  if isinstance(action, dict):
    return [action]
  return action


class ToolEnvironment(base_environment.BaseTaskEnv):

  def __init__(self, task: Optional[Dict[str, Any]] = None, *, tool_map: Dict[str, Type[base_tool.BaseTool]],
               reward_fn=None, max_steps: int = 10, **kwargs):
    if reward_fn is None:
      logging.warning("No reward_fn provided, skipping trajectory reward computation.")
    super().__init__(task=task, reward_fn=reward_fn, max_steps=max_steps, **kwargs)
    self.tool_manager = tool_manager.ToolManager(tool_map)

  def _initial_observation(self) -> Dict[str, Any]:
    return self.task

  @staticmethod
  def _finish_call(calls: Any) -> Optional[Dict[str, Any]]:
    if not isinstance(calls, list):
      return None
    return next((c for c in calls if c.get("function", {}).get("name") == FINISH), None)

  @classmethod
  def _extract_llm_answer(cls, action: Any) -> str:
    if isinstance(action, str):
      return action
    fin = cls._finish_call(action)
    if fin is None:
      return str(action)
    args = _arguments(fin)
    return args if isinstance(args, str) else args.get("response", "")

  def _step_impl(self, action: Any) -> base_environment.EnvStepResult:
    calls = _calls_of(action)
    if isinstance(calls, str) or self._finish_call(calls) is not None:
      return self.final(self._extract_llm_answer(calls), response=calls)
    return self.turn({"tool_outputs": self._execute_tool_calls(calls)}, response=calls)

  def _execute_tool_calls(self, tool_calls: List[Dict[str, Any]]) -> Dict[str, str]:
    batch = []
    for call in tool_calls:
      args = call["function"]["arguments"]
      request = base_tool.ToolCall(name=call["function"]["name"], arguments=json.loads(args) if isinstance(args, str) else args)
      request.id = call.get("id") or str(uuid.uuid4())
      batch.append(request)
    return self.tool_manager.execute_calls(batch, parallel=True)

  @classmethod
  def from_dict(cls, env_args: Dict[str, Any]) -> "ToolEnvironment":
    """`env_args` is the task record with `tool_map`, `reward_fn` and `max_steps` mixed in."""
    record = dict(env_args)
    return cls(tool_map=record.pop("tool_map", None), reward_fn=record.pop("reward_fn", None),
               max_steps=record.pop("max_steps", 10), task=record)
