"""Tool interface (tunix/rl/agentic/tools/base_tool.py:30-216).

A tool has a name, a one-line description, an OpenAI function-calling schema and an `apply` (or `apply_async`)
that returns a `ToolOutput`. Instances are shared between concurrent episodes, so they are frozen once the
outermost constructor returns (`utils.immutable.FrozenAfterInit`).
`FunctionTool` turns a plain Python function into a tool, deriving the parameter schema from its signature.
"""
from __future__ import annotations

import abc
import dataclasses
import functools
import inspect
import json
from typing import Any, Callable, Dict, List, Optional, Union

from ....utils import immutable


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

  def render(self) -> str:
    """What the model reads: the error if there is one, JSON for structured output, else the text."""
    if self.error:
      return f"Error: {self.error}"
    if self.output is None:
      return ""
    return json.dumps(self.output) if isinstance(self.output, (dict, list)) else str(self.output)

  __repr__ = __str__ = render


def function_schema(name: str, description: str, parameters: Optional[Dict[str, Any]] = None) -> Dict[str, Any]:
  return {"type": "function", "function": {"name": name, "description": description,
                                           "parameters": parameters if parameters is not None else {}}}


class BaseTool(immutable.FrozenAfterInit, abc.ABC):

  def __init__(self, name: str, description: str):
    self.name = name
    self.description = description
    super().__init__()

  @abc.abstractmethod
  def get_json_schema(self) -> Dict[str, Any]:
    """OpenAI function-calling schema: {"type": "function", "function": {name, description, parameters}}."""

  def to_mcp_json(self) -> Dict[str, Any]:
    return function_schema(self.name, self.description, getattr(self, "inputSchema", {}))

  def apply(self, **kwargs) -> ToolOutput:
    raise NotImplementedError("Tool must implement either `apply()` or `apply_async()`")

  async def apply_async(self, **kwargs) -> ToolOutput:
    raise NotImplementedError("Tool must implement either `apply()` or `apply_async()`")


_JSON_TYPES = {int: "integer", float: "number", bool: "boolean", str: "string", list: "array", dict: "object"}


class FunctionTool(BaseTool):
  """A tool made from a function: parameters and their JSON types come from the signature, the description
  from the first docstring line (unless given), the output is whatever the function returns."""

  def __init__(self, fn: Callable[..., Any], name: Optional[str] = None, description: Optional[str] = None):
    super().__init__(name or fn.__name__, description or (inspect.getdoc(fn) or "").split("\n")[0])
    self.fn = fn
    props, required = {}, []
    for pname, p in inspect.signature(fn).parameters.items():
      if p.kind in (p.VAR_POSITIONAL, p.VAR_KEYWORD):
        continue
      props[pname] = {"type": _JSON_TYPES.get(p.annotation, "string")}
      if p.default is p.empty:
        required.append(pname)
    self.inputSchema = {"type": "object", "properties": props, "required": required}

  def get_json_schema(self) -> Dict[str, Any]:
    return self.to_mcp_json()

  def apply(self, **kwargs) -> ToolOutput:
    return ToolOutput(name=self.name, output=self.fn(**kwargs))
