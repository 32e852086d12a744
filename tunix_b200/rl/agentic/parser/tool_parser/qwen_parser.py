"""Qwen tool-call format: `<tool_call>{"name": ..., "arguments": {...}}</tool_call>`
(tunix/rl/agentic/parser/tool_parser/qwen_parser.py:30-120)."""
from __future__ import annotations

import json
import logging
import re
from typing import Any, Dict, List

from ...tools import base_tool
from . import tool_parser_base

_CALL = re.compile(r"<tool_call>(.*?)</tool_call>", re.S)


class QwenToolParser(tool_parser_base.ToolParser):
  tool_call_begin, tool_call_end = "<tool_call>", "</tool_call>"
  tool_output_begin, tool_output_end = "<tool_response>", "</tool_response>"

  def parse_qwen_tool_calls(self, text: str) -> List[Dict[str, Any]]:
    calls = []
    for body in _CALL.findall(text):
      try:
        d = json.loads(body.strip())
        calls.append({"name": d["name"], "arguments": d["arguments"]})
      except (json.JSONDecodeError, KeyError, TypeError):
        logging.warning("Error parsing tool call: %s", body.strip())
    return calls

  def parse(self, model_response: str) -> List[base_tool.ToolCall]:
    return [base_tool.ToolCall(**c) for c in self.parse_qwen_tool_calls(model_response)]

  def get_tool_prompt(self, tools: List[base_tool.BaseTool], schema_style: str = "openai") -> str:
    schema = self._tools_schema_dump(tools, schema_style=schema_style)
    return ("You are provided with function signatures within <tools></tools> XML tags:\n<tools>\n" + schema +
            "\n</tools>\nFor each function call, return a json object with function name and arguments within "
            "<tool_call></tool_call> XML tags:\n<tool_call>\n"
            '{"name": "<function-name>", "arguments": <args-json-object>}\n</tool_call>')
