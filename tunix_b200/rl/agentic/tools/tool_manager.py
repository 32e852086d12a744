"""Registry and executor of tools (tunix/rl/agentic/tools/tool_manager.py:28-234).

Tools are built once from a `{name: class}` map (the description is the first docstring line of the class) or
added ready-made (`register_mcp_tool`). Every way of running a tool goes through `_guarded`, which turns an
unknown name or an exception into a `ToolOutput` with `error` set - a failing tool is something the model has to
deal with, not the episode. `execute_calls` runs the calls of one turn on a thread pool and returns their rendered
outputs in call order."""
from __future__ import annotations

import inspect
import uuid
from concurrent import futures
from typing import Any, Awaitable, Callable, Dict, List, Type, Union

from . import base_tool

_MAX_PARALLEL_CALLS = 16


def _first_doc_line(cls: type, fallback: str) -> str:
  return (inspect.getdoc(cls) or fallback or "").strip().split("\n")[0]


class ToolManager:

  def __init__(self, tool_map: Dict[str, Type[base_tool.BaseTool]], *, desc_fallback: str = ""):
    self._tool_dict: Dict[str, base_tool.BaseTool] = {}
    for name, cls in tool_map.items():
      if inspect.isabstract(cls):
        raise TypeError(f"Cannot instantiate abstract tool class '{name}': {cls.__name__}. Implement "
                        "get_json_schema() and apply() or apply_async().")
      self._tool_dict[name] = cls(name=name, description=_first_doc_line(cls, desc_fallback))

  # ---- registry
  @property
  def names(self) -> List[str]:
    return list(self._tool_dict)

  def get_tools(self) -> List[base_tool.BaseTool]:
    return list(self._tool_dict.values())

  def register_mcp_tool(self, tool: base_tool.BaseTool) -> None:
    self._tool_dict[tool.name] = tool

  def get_json_schema(self) -> List[Dict[str, Any]]:
    return [tool.get_json_schema() for tool in self.get_tools()]

  def get_mcp_schema(self) -> List[Dict[str, Any]]:
    return [tool.to_mcp_json() for tool in self.get_tools()]

  # ---- running one tool
  def _guarded(self, tool_name: str, invoke: Callable[[base_tool.BaseTool], Any]) -> Any:
    """invoke(tool), or an error output when the tool is unknown or raises (NotImplementedError passes)."""
    tool = self._tool_dict.get(tool_name)
    if tool is None:
      return base_tool.ToolOutput(name=tool_name, error=f"Tool '{tool_name}' not registered.")
    try:
      return invoke(tool)
    except NotImplementedError:
      raise
    except Exception as e:          # noqa: BLE001 - reported to the model
      return base_tool.ToolOutput(name=tool_name, error=f"{type(e).__name__}: {e}")

  def run(self, tool_name: str, **kwargs: Any) -> base_tool.ToolOutput:
    try:
      return self._guarded(tool_name, lambda tool: tool.apply(**kwargs))
    except NotImplementedError as e:
      return base_tool.ToolOutput(name=tool_name, error=f"{type(e).__name__}: {e}")

  async def run_async(self, tool_name: str, **kwargs: Any) -> base_tool.ToolOutput:
    """The tool's coroutine where it has one, else its blocking `apply`."""
    try:
      pending: Union[base_tool.ToolOutput, Awaitable[base_tool.ToolOutput]] = self._guarded(
          tool_name, lambda tool: tool.apply_async(**kwargs))
      if not inspect.isawaitable(pending):
        return pending
      return await pending
    except NotImplementedError:
      return self.run(tool_name, **kwargs)
    except Exception as e:          # noqa: BLE001
      return base_tool.ToolOutput(name=tool_name, error=f"{type(e).__name__}: {e}")

  # ---- running the calls of one turn
  def execute_calls(self, calls: List[base_tool.ToolCall], parallel: bool = True) -> Dict[str, str]:
    """-> {call id: output rendered as a string}, in call order; ids come from the calls or are generated."""
    ids = [getattr(call, "id", None) or str(uuid.uuid4()) for call in calls]

    def one(call: base_tool.ToolCall) -> str:
      try:
        return str(self.run(tool_name=call.name, **call.arguments))
      except Exception as e:        # noqa: BLE001 - e.g. arguments that are not a mapping
        return f"Error: {type(e).__name__}: {e}"

    if parallel and len(calls) > 1:
      with futures.ThreadPoolExecutor(max_workers=min(len(calls), _MAX_PARALLEL_CALLS)) as pool:
        rendered = list(pool.map(one, calls))
    else:
      rendered = [one(call) for call in calls]
    return dict(zip(ids, rendered))
