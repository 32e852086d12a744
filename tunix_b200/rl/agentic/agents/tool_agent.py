"""Tool-calling agent (tunix/rl/agentic/agents/tool_agent.py:32-160).

The system prompt carries the tool schemas rendered by the model family's tool parser. Each model response is
parsed for tool calls; a response without a parsable call is taken as the final answer and wrapped in a call to
the pseudo-tool `finish`. Observations come back either as tool outputs (one `tool` message per call id) or as
a new user turn."""
from __future__ import annotations

import copy
import json
import logging
import uuid
from typing import Any, Dict, List, Optional, Type

from ..parser.tool_parser import tool_parser_registry
from ..tools import base_tool, tool_manager
from . import agent_types, base_agent

_USER_KEYS = ("question", "prompts")


def wire_call(name: str, arguments: Any) -> Dict[str, Any]:
  """One call in the OpenAI wire format, with a fresh id."""
  return {"id": str(uuid.uuid4()), "type": "function", "function": {"name": name, "arguments": arguments}}


class ToolAgent(base_agent.ConversationAgentBase):

  def __init__(self, system_prompt: str, tool_parser_name: str = "qwen",
               tool_map: Optional[Dict[str, Type[base_tool.BaseTool]]] = None):
    self.tool_manager = tool_manager.ToolManager(tool_map=tool_map or {})
    self.tool_parser = tool_parser_registry.get_tool_parser(tool_parser_name)()
    self.tools_prompt = self.tool_parser.get_tool_prompt(self.tool_manager.get_tools())
    super().__init__(system_prompt=system_prompt)

  def _init_messages(self, system_prompt: str) -> None:
    self._messages = [{"role": "system", "content": (system_prompt or "") + (self.tools_prompt or "")}]

  # ---- environment -> conversation
  def _observation_to_messages(self, observation: Any, reward: float, done: bool, info: Dict[str, Any]) -> None:
    if isinstance(observation, str):
      self._messages.append({"role": "user", "content": observation})
      return
    if not isinstance(observation, dict):
      return
    outputs = observation.get("tool_outputs")
    if outputs is not None:
      self._messages.extend({"role": "tool", "tool_call_id": call_id, "content": "Tool returned result: " + (text or "")}
                            for call_id, text in outputs.items())
      return
    key = next((k for k in _USER_KEYS if k in observation), None)
    if key is None:
      logging.warning("Unknown dict observation format: %s", observation)
      return
    self._messages.append({"role": "user", "content": self._text(observation[key])})

  # ---- model -> action
  def _calls_in(self, response: str) -> List[Dict[str, Any]]:
    try:
      parsed = self.tool_parser.parse(response)
    except Exception as e:  # noqa: BLE001 - a malformed call is the model's problem, not the episode's
      logging.warning("ToolParser failed: %s", e)
      parsed = []
    if not parsed:
      return [wire_call("finish", {"response": response})]
    return [wire_call(c.name, json.dumps(c.arguments) if isinstance(c.arguments, dict) else c.arguments) for c in parsed]

  def update_from_model(self, response: str, **kwargs) -> agent_types.Action:
    action = agent_types.Action(action=self._calls_in(response))
    self._messages.append({"role": "assistant", "content": response})
    self._trajectory.steps.append(agent_types.Step(chat_completions=copy.deepcopy(self._messages),
                                                   action=agent_types.Action(action=action.action),
                                                   model_response=response))
    return action
