"""Tool interface (tunix/rl/agentic/tools/base_tool.py:30-216). Tools are stateless and frozen
after construction, so one instance can serve concurrent episodes."""
from __future__ import annotations

import abc
import dataclasses
import json
from typing import Any, Dict, List, Optional, Union


@dataclasses.dataclass
class ToolCall:
  name: str
  arguments: Dict[str, Any]


@dataclasses.dataclass
class ToolOutput:
  name: str
  output: Optional[Union[str, List[Any], Dict[str, Any]]] = None
  error: Optional[str] = None
  metadata: Optional[Dict[str, Any]] = None

  def __repr__(self) -> str:
    if self.error:
      return f"Error: {self.error}"
    if self.output is None:
      return ""
    if isinstance(self.output, (dict, list)):
      return json.dumps(self.output)
    return str(self.output)

  __str__ = __repr__


class _FreezeAfterInit(abc.ABCMeta):
  def __call__(cls, *a, **k):
    obj = super().__call__(*a, **k)
    object.__setattr__(obj, "_locked", True)
    return obj


class BaseTool(metaclass=_FreezeAfterInit):
  def __init__(self, name: str, description: str):
    self.name = name
    self.description = description

  def __setattr__(self, name: str, value: Any):
    if getattr(self, "_locked", False):
      raise AttributeError(f"Cannot modify immutable {self.__class__.__name__} instance after initialization "
                           f"(attempted to set '{name}')")
    object.__setattr__(self, name, value)

  @abc.abstractmethod
  def get_json_schema(self) -> Dict[str, Any]:
    """OpenAI function-calling schema: {"type": "function", "function": {name, description, parameters}}."""

  def to_mcp_json(self) -> Dict[str, Any]:
    return {"type": "function", "function": {"name": self.name, "description": self.description,
                                             "parameters": getattr(self, "inputSchema", {})}}

  def apply(self, **kwargs) -> ToolOutput:
    raise NotImplementedError("Tool must implement either `apply()` or `apply_async()`")

  async def apply_async(self, **kwargs) -> ToolOutput:
    raise NotImplementedError("Tool must implement either `apply()` or `apply_async()`")
