"""Tool-calling agent (tunix/rl/agentic/agents/tool_agent.py:32-160): the system prompt carries
the tool schemas rendered by the parser; a response with no parsable call becomes a `finish`
call carrying the raw response."""
from __future__ import annotations

import copy
import json
import logging
import uuid
from typing import Any, Dict, Optional, Type

from ..parser.tool_parser import tool_parser_registry
from ..tools import base_tool, tool_manager
from . import agent_types, base_agent


class ToolAgent(base_agent.ConversationAgentBase):
  def __init__(self, system_prompt: str, tool_parser_name: str = "qwen",
               tool_map: Optional[Dict[str, Type[base_tool.BaseTool]]] = None):
    self.tool_manager = tool_manager.ToolManager(tool_map=tool_map or {})
    self.tool_parser = tool_parser_registry.get_tool_parser(tool_parser_name)()
    self.tools_prompt = self.tool_parser.get_tool_prompt(self.tool_manager.get_tools())
    super().__init__(system_prompt=system_prompt)

  def _init_messages(self, system_prompt: str) -> None:
    self._messages = [{"role": "system", "content": (system_prompt or "") + (self.tools_prompt or "")}]

  def _observation_to_messages(self, observation: Any, reward: float, done: bool, info: Dict[str, Any]) -> None:
    if isinstance(observation, dict):
      if "tool_outputs" in observation:
        for call_id, output in observation["tool_outputs"].items():
          self._messages.append({"role": "tool", "tool_call_id": call_id,
                                 "content": "Tool returned result: " + (output or "")})
      elif "question" in observation or "prompts" in observation:
        key = "question" if "question" in observation else "prompts"
        self._messages.append({"role": "user", "content": self._text(observation[key])})
      else:
        logging.warning("Unknown dict observation format: %s", observation)
    elif isinstance(observation, str):
      self._messages.append({"role": "user", "content": observation})

  def update_from_model(self, response: str, **kwargs) -> agent_types.Action:
    try:
      calls = self.tool_parser.parse(response)
    except Exception as e:  # a malformed call is the model's problem, not the episode's
      logging.warning("ToolParser failed: %s", e)
      calls = []
    if not calls:
      payload = [{"id": str(uuid.uuid4()), "type": "function",
                  "function": {"name": "finish", "arguments": {"response": response}}}]
    else:
      payload = [{"id": str(uuid.uuid4()), "type": "function",
                  "function": {"name": c.name, "arguments": json.dumps(c.arguments) if isinstance(c.arguments, dict)
                               else c.arguments}} for c in calls]
    self._messages.append({"role": "assistant", "content": response})
    self._trajectory.steps.append(agent_types.Step(chat_completions=copy.deepcopy(self._messages),
                                                   action=agent_types.Action(action=payload),
                                                   model_response=response))
    return agent_types.Action(action=payload)
