"""Gemini function calling is structured on the API side, so there is nothing to parse from text
(tunix/rl/agentic/parser/tool_parser/gemini_parser.py:27-38)."""
from __future__ import annotations

from typing import Any, List

from ...tools import base_tool
from . import tool_parser_base


class GeminiToolParser(tool_parser_base.ToolParser):
  def parse(self, model_response: Any) -> List[base_tool.ToolCall]:
    return []

  def get_tool_prompt(self, tools: List[base_tool.BaseTool], *, schema_style: str = "gemini") -> str:
    return "Return a functionCall with name and args."
