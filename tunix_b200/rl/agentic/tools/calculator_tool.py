"""Four-function calculator tool (tunix/rl/agentic/tools/calculator_tool.py:25-131)."""
from __future__ import annotations

import operator
from typing import Any, Dict

from . import base_tool

_OPS = {"+": operator.add, "-": operator.sub, "*": operator.mul, "/": operator.truediv}


class CalculatorTool(base_tool.BaseTool):
  def get_json_schema(self) -> Dict[str, Any]:
    return {"type": "function", "function": {
        "name": self.name, "description": self.description,
        "parameters": {"type": "object", "required": ["a", "b", "op"], "properties": {
            "a": {"type": "number", "description": "The first operand"},
            "b": {"type": "number", "description": "The second operand"},
            "op": {"type": "string", "enum": list(_OPS), "description": "Operator, one of: + - * /"}}}}}

  def apply(self, **kwargs: Any) -> base_tool.ToolOutput:
    a, b, op = kwargs.get("a"), kwargs.get("b"), kwargs.get("op")
    err = None
    if a is None or b is None or op is None:
      err = "Missing required arguments: 'a', 'b', and 'op'"
    elif isinstance(a, bool) or isinstance(b, bool) or not isinstance(a, (int, float)) or not isinstance(b, (int, float)):
      err = "Operands 'a' and 'b' must be numbers (int or float)"
    elif not isinstance(op, str):
      err = "Operator 'op' must be a string"
    elif op not in _OPS:
      err = f"Unsupported operator: {op}. Use one of: + - * /"
    elif op == "/" and b == 0:
      err = "Division by zero is not allowed"
    if err:
      return base_tool.ToolOutput(name=self.name, error=err)
    try:
      return base_tool.ToolOutput(name=self.name, output=_OPS[op](a, b))
    except Exception as e:  # overflow and the like
      return base_tool.ToolOutput(name=self.name, error=f"{type(e).__name__}: {e}")
