"""Tool-call parser interface (tunix/rl/agentic/parser/tool_parser/tool_parser_base.py:27-98)."""
from __future__ import annotations

import abc
import json
from typing import Any, Dict, List

from ...tools import base_tool


class ToolParser(abc.ABC):
  @abc.abstractmethod
  def parse(self, model_response: str) -> List[base_tool.ToolCall]: ...

  @abc.abstractmethod
  def get_tool_prompt(self, tools: List[base_tool.BaseTool], *, schema_style: str = "openai") -> str: ...

  def _tools_schema_dump(self, tools: List[base_tool.BaseTool], *, schema_style: str = "openai") -> str:
    if schema_style == "openai":
      schemas = [t.get_json_schema() for t in tools]
    elif schema_style == "mcp":
      schemas = [t.to_mcp_json() for t in tools]
    elif schema_style == "gemini":
      schemas = [t.get_json_schema().get("function", {}) for t in tools]
    else:
      raise ValueError(f"Unknown schema_style: {schema_style}")
    return json.dumps(schemas, ensure_ascii=False, indent=2)

  def parse_tool_outputs(self) -> Dict[str, Any]:
    return {}
