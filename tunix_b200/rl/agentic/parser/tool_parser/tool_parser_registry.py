"""Tool parsers by name."""
from __future__ import annotations

from typing import Dict, Type

from . import gemini_parser, qwen_parser, tool_parser_base

_PARSERS: Dict[str, Type[tool_parser_base.ToolParser]] = {"qwen": qwen_parser.QwenToolParser,
                                                          "gemini": gemini_parser.GeminiToolParser}


def register_tool_parser(name: str, cls: Type[tool_parser_base.ToolParser]) -> None:
  _PARSERS[name] = cls


def get_tool_parser(parser_name: str = "qwen") -> Type[tool_parser_base.ToolParser]:
  if parser_name not in _PARSERS:
    raise ValueError(f"Unknown parser: {parser_name}")
  return _PARSERS[parser_name]
