"""Multi-turn tool environment (tunix/rl/agentic/environments/tool_environment.py:36-248): an
action is a final answer (string, or a `finish` call) that ends the episode and is scored, or a
list of tool calls whose outputs become the next observation."""
from __future__ import annotations

import json
import logging
import uuid
from typing import Any, Dict, List, Optional, Type

from ..agents import agent_types
from ..tools import base_tool, tool_manager
from . import base_environment


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
  def _is_finish(call: Dict[str, Any]) -> bool:
    return call.get("function", {}).get("name") == "finish"

  def _step_impl(self, action: Any) -> base_environment.EnvStepResult:
    if isinstance(action, agent_types.Action):
      action = action.action
    if action is None:
      action = []
    if isinstance(action, dict):
      action = [action]
    done = isinstance(action, str) or (isinstance(action, list) and any(self._is_finish(c) for c in action))
    if done:
      answer = self._extract_llm_answer(action)
      reward = self.reward_fn(task=self.task, action=answer) if self.reward_fn is not None else 0.0
      return base_environment.EnvStepResult(observation={}, reward=reward, done=True, info={"response": action})
    return base_environment.EnvStepResult(observation={"tool_outputs": self._execute_tool_calls(action)}, reward=0.0,
                                          done=False, info={"response": action})

  @staticmethod
  def _extract_llm_answer(action: Any) -> str:
    if isinstance(action, str):
      return action
    if isinstance(action, list):
      for call in action:
        if ToolEnvironment._is_finish(call):
          args = call["function"].get("arguments", {})
          if isinstance(args, str):
            try:
              args = json.loads(args)
            except json.JSONDecodeError:
              return args
          return args.get("response", "")
    return str(action)

  def _execute_tool_calls(self, tool_calls: List[Dict[str, Any]]) -> Dict[str, str]:
    objs = []
    for tc in tool_calls:
      args = tc["function"]["arguments"]
      if isinstance(args, str):
        args = json.loads(args)
      obj = base_tool.ToolCall(name=tc["function"]["name"], arguments=args)
      obj.id = tc.get("id") or str(uuid.uuid4())
      objs.append(obj)
    return self.tool_manager.execute_calls(objs, parallel=True)

  @classmethod
  def from_dict(cls, env_args: Dict[str, Any]) -> "ToolEnvironment":
    env_args = dict(env_args)
    tool_map = env_args.pop("tool_map", None)
    reward_fn = env_args.pop("reward_fn", None)
    max_steps = env_args.pop("max_steps", 10)
    return cls(task=env_args, tool_map=tool_map, reward_fn=reward_fn, max_steps=max_steps)
