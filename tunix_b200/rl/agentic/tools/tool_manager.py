"""Registry and executor of tools (tunix/rl/agentic/tools/tool_manager.py:28-234)."""
from __future__ import annotations

import inspect
import uuid
from concurrent import futures
from typing import Any, Dict, List, Optional, Type

from . import base_tool


class ToolManager:
  def __init__(self, tool_map: Dict[str, Type[base_tool.BaseTool]], *, desc_fallback: str = ""):
    self._tool_dict: Dict[str, base_tool.BaseTool] = {}
    for name, cls in tool_map.items():
      if inspect.isabstract(cls):
        raise TypeError(f"Cannot instantiate abstract tool class '{name}': {cls.__name__}. Implement "
                        "get_json_schema() and apply() or apply_async().")
      desc = (inspect.getdoc(cls) or desc_fallback or "").strip().split("\n")[0]
      self._tool_dict[name] = cls(name=name, description=desc)

  @property
  def names(self) -> List[str]:
    return list(self._tool_dict)

  def get_tools(self) -> List[base_tool.BaseTool]:
    return list(self._tool_dict.values())

  def get_json_schema(self) -> List[Dict[str, Any]]:
    return [t.get_json_schema() for t in self._tool_dict.values()]

  def get_mcp_schema(self) -> List[Dict[str, Any]]:
    return [t.to_mcp_json() for t in self._tool_dict.values()]

  def register_mcp_tool(self, tool: base_tool.BaseTool) -> None:
    self._tool_dict[tool.name] = tool

  def run(self, tool_name: str, **kwargs: Any) -> base_tool.ToolOutput:
    tool = self._tool_dict.get(tool_name)
    if tool is None:
      return base_tool.ToolOutput(name=tool_name, error=f"Tool '{tool_name}' not registered.")
    try:
      return tool.apply(**kwargs)
    except Exception as e:
      return base_tool.ToolOutput(name=tool_name, error=f"{type(e).__name__}: {e}")

  async def run_async(self, tool_name: str, **kwargs: Any) -> base_tool.ToolOutput:
    tool = self._tool_dict.get(tool_name)
    if tool is None:
      return base_tool.ToolOutput(name=tool_name, error=f"Tool '{tool_name}' not registered.")
    try:
      return await tool.apply_async(**kwargs)
    except NotImplementedError:
      return self.run(tool_name, **kwargs)
    except Exception as e:
      return base_tool.ToolOutput(name=tool_name, error=f"{type(e).__name__}: {e}")

  def execute_calls(self, calls: List[base_tool.ToolCall], parallel: bool = True) -> Dict[str, str]:
    """-> {call id: output rendered as a string}; ids come from the calls or are generated."""
    ids = [getattr(c, "id", None) or str(uuid.uuid4()) for c in calls]
    if not parallel or len(calls) <= 1:
      return {cid: str(self.run(tool_name=c.name, **c.arguments)) for cid, c in zip(ids, calls)}
    out: Dict[str, str] = {}
    with futures.ThreadPoolExecutor() as ex:
      futs = {ex.submit(self.run, tool_name=c.name, **c.arguments): cid for cid, c in zip(ids, calls)}
      for f in futures.as_completed(futs):
        try:
          out[futs[f]] = str(f.result())
        except Exception as e:
          out[futs[f]] = f"Error: {type(e).__name__}: {e}"
    return out
