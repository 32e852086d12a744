"""From whatever an agent calls an "action" to a list of schema `ToolCall`s
(tunix/experimental/trajectory/action_converter.py:15-379).

Agents hand over actions in many shapes: an `Action` wrapper (possibly nested), a `ToolCall` already, an OpenAI
message part (`{"id", "type": "function", "function": {"name", "arguments"}}`), an Anthropic part
(`{"type": "tool_use", "name", "input"}`), a flat `{"name", "args"}` dict, a bare dict of arguments, an object
with such attributes, a JSON string, or model text with `<tool_call>` / `<function=...>` / `<invoke name=...>`
markup. `extract_tool_calls` unwraps the action and runs the payload through *recognisers* in a fixed order; the
first that understands it wins. Scalars and arrays (discrete or continuous control actions) are not tool calls.
Calls without an id are numbered `call_1, call_2, ...` in order of appearance.
"""
from __future__ import annotations

import dataclasses
import json
import logging
import re
from typing import Any, Callable, Dict, Iterable, List, Mapping, Optional, Sequence

import numpy as np

from ...rl.agentic.agents import agent_types
from . import trajectory as trajectory_lib

ToolCall = trajectory_lib.ToolCall
log = logging.getLogger(__name__)

# the same field under the names different APIs give it, most common first
ID_ALIASES = ("id", "tool_call_id", "call_id", "function_id")
NAME_ALIASES = ("name", "function_name", "tool_name", "func", "function")
ARGUMENT_ALIASES = ("arguments", "args", "parameters", "params", "input", "inputs")
_ENVELOPE = frozenset(ID_ALIASES + NAME_ALIASES + ("type",))
_NOT_A_CALL = (bool, int, float, np.number, np.ndarray)
DEFAULT_FUNCTION = "action"


class _Numbering:
  """`call_<n>` ids for calls that carry none; n counts the calls produced so far."""

  def __init__(self, produced: int = 0):
    self.produced = produced

  def next_id(self) -> str:
    return f"call_{self.produced + 1}"

  def emit(self, name: Any, arguments: Any, call_id: Any = None) -> ToolCall:
    call = ToolCall(tool_call_id=str(call_id or self.next_id()), function_name=str(name or DEFAULT_FUNCTION),
                    arguments=as_arguments(arguments))
    self.produced += 1
    return call


def _first(source: Any, aliases: Sequence[str]) -> Any:
  """First alias with a non-None value, looked up as key (mappings) or attribute (objects)."""
  for alias in aliases:
    value = source.get(alias) if isinstance(source, Mapping) else getattr(source, alias, None)
    if value is not None:
      return value
  return None


def strip_code_fence(text: str) -> str:
  """Drops a surrounding markdown fence (```json ... ```), if there is one."""
  body = text.strip()
  if not body.startswith("```"):
    return body
  lines = body.splitlines()[1:]
  if lines and lines[-1].strip() == "```":
    lines.pop()
  return "\n".join(lines).strip()


def as_mapping(obj: Any) -> Optional[Dict[str, Any]]:
  """A dict view of dicts, objects with `to_dict()`, dataclass instances and plain objects; None otherwise."""
  if isinstance(obj, dict):
    return obj
  if isinstance(obj, type):
    return None
  exporter = getattr(obj, "to_dict", None)
  if callable(exporter):
    exported = exporter()
    if isinstance(exported, dict):
      return exported
  if dataclasses.is_dataclass(obj):
    return dataclasses.asdict(obj)
  if hasattr(obj, "__dict__"):
    return dict(vars(obj))
  return None


def _json_or_none(text: str, what: str) -> Any:
  try:
    return json.loads(text)
  except ValueError as e:
    log.warning("Failed to parse %s: %s", what, e)
    return None


def as_arguments(raw: Any) -> Dict[str, Any]:
  """Arguments as a dict: mappings and objects as they are, strings parsed as JSON objects, anything else {}."""
  if raw is None:
    return {}
  mapped = as_mapping(raw)
  if mapped is not None:
    return mapped
  if isinstance(raw, str) and strip_code_fence(raw):
    parsed = _json_or_none(strip_code_fence(raw), "arguments JSON string")
    if isinstance(parsed, dict):
      return parsed
  return {}


# ----------------------------------------------------------------------------------- mappings and objects
def _rest(mapping: Mapping[str, Any]) -> Dict[str, Any]:
  return {k: v for k, v in mapping.items() if k not in _ENVELOPE}


def call_from_mapping(item: Mapping[str, Any], numbering: _Numbering) -> Optional[ToolCall]:
  """One call out of a dict in OpenAI, Anthropic or flat form; a dict that is neither is taken as the arguments
  of a call to `action`, and a dict that holds nothing but an id / type is no call at all."""
  call_id = _first(item, ID_ALIASES)
  nested = item.get("function")
  if isinstance(nested, dict):                                   # OpenAI: the call sits under "function"
    args = _first(nested, ARGUMENT_ALIASES)
    if args is None and len(nested) > 1:
      args = _rest(nested)
    return numbering.emit(_first(nested, NAME_ALIASES), args, call_id)
  name, args = _first(item, NAME_ALIASES), _first(item, ARGUMENT_ALIASES)
  if item.get("type") == "tool_use":                             # Anthropic
    if args is None and len(item) > 2:
      args = _rest(item)
    return numbering.emit(name, args, call_id)
  if args is None and name is not None:                          # flat: the other keys are the arguments
    args = _rest(item)
  elif args is None:
    payload_keys = [k for k in item if k not in ID_ALIASES and k != "type"]
    if item and not payload_keys:
      return None
    args = item                                                  # bare arguments
  return numbering.emit(name, args, call_id)


def call_from_item(item: Any, numbering: _Numbering) -> Optional[ToolCall]:
  if item is None or isinstance(item, _NOT_A_CALL):
    return None
  if isinstance(item, ToolCall):
    numbering.produced += 1
    return item
  mapped = as_mapping(item)
  if mapped is not None:
    return call_from_mapping(mapped, numbering)
  name = _first(item, NAME_ALIASES)                              # slotted objects and the like
  if name is None:
    return None
  return numbering.emit(name, _first(item, ARGUMENT_ALIASES), _first(item, ID_ALIASES))


# ----------------------------------------------------------------------------------- text
_XML_CALL = re.compile(r"<(?:function|invoke)(?:\s*=\s*|\s+name=\s*)([^>]+)>(.*?)(?:</(?:function|invoke)>|$)", re.DOTALL)
_XML_PARAM = re.compile(r"<parameter(?:\s*=\s*|\s+name=\s*)([^>]+)>(.*?)(?:</parameter>|$)", re.DOTALL)
_WRAPPED = re.compile(r"<(?:tool_call|function_call)>(.*?)(?:</(?:tool_call|function_call)>|$)", re.DOTALL)
_TAG_NAME = re.compile(r"<(?:name|function_name)>(.*?)</(?:name|function_name)>", re.DOTALL)
_TAG_ARGS = re.compile(r"<(?:arguments|parameters|args|params|input)>(.*?)</(?:arguments|parameters|args|params|input)>",
                       re.DOTALL)


def _unquote(text: str) -> str:
  return text.strip().strip("\"'")


def calls_from_xml(text: str, numbering: _Numbering) -> List[ToolCall]:
  """`<function=NAME>...</function>` / `<invoke name="NAME">...</invoke>` blocks. The body is `<parameter=K>V`
  pairs, a JSON object, or free text (kept under "input")."""
  calls = []
  for found in _XML_CALL.finditer(text):
    name, body = _unquote(found.group(1)), found.group(2).strip()
    if not name:
      continue
    params = _XML_PARAM.findall(body)
    unfenced = strip_code_fence(body)
    if params:
      args: Any = {_unquote(k): v.strip() for k, v in params}
    elif unfenced.startswith("{"):
      parsed = _json_or_none(unfenced, "XML function body JSON")
      args = parsed if isinstance(parsed, dict) else {}
    else:
      args = {"input": body} if body else {}
    calls.append(numbering.emit(name, args, numbering.next_id()))
  return calls


def _calls_from_wrapped_block(block: str, numbering: _Numbering) -> List[ToolCall]:
  """The inside of one `<tool_call>` element: JSON, `<name>` / `<arguments>` tags, or function XML."""
  inner = strip_code_fence(block.strip())
  if not inner:
    return []
  if inner.startswith(("{", "[")):
    parsed = _json_or_none(inner, "tool call block JSON")
    if isinstance(parsed, dict):
      call = call_from_mapping(parsed, numbering)
      if call is not None:
        return [call]
    elif isinstance(parsed, list):
      calls = calls_from_payload(parsed, numbering)
      if calls:
        return calls
  name = _TAG_NAME.search(inner)
  if name is not None:
    args = _TAG_ARGS.search(inner)
    return [numbering.emit(name.group(1).strip(), args.group(1).strip() if args else "{}", numbering.next_id())]
  if "<function" in inner or "<invoke" in inner:
    return calls_from_xml(inner, numbering)
  return []


def calls_from_text(text: str, numbering: _Numbering) -> List[ToolCall]:
  body = text.strip()
  if not body:
    return []
  unfenced = strip_code_fence(body)
  if unfenced.startswith(("{", "[")):                            # the whole string is JSON
    parsed = _json_or_none(unfenced, "JSON tool calls string")
    if isinstance(parsed, (dict, list)):
      calls = calls_from_payload(parsed, numbering)
      if calls:
        return calls
  if "<tool_call>" in body or "<function_call>" in body:          # wrapped blocks inside prose
    calls = []
    for block in _WRAPPED.findall(body):
      calls.extend(_calls_from_wrapped_block(block, numbering))
    if calls:
      return calls
  if "<function" in body or "<invoke" in body:
    return calls_from_xml(body, numbering)
  return []


# ----------------------------------------------------------------------------------- dispatch
def calls_from_payload(payload: Any, numbering: Optional[_Numbering] = None) -> List[ToolCall]:
  numbering = numbering or _Numbering()
  if payload is None or isinstance(payload, _NOT_A_CALL):
    return []
  if isinstance(payload, str):
    return calls_from_text(payload, numbering)
  if isinstance(payload, (list, tuple)):
    calls: List[ToolCall] = []
    for item in payload:
      if isinstance(item, str):
        calls.extend(calls_from_text(item, numbering))
      else:
        call = call_from_item(item, numbering)
        if call is not None:
          calls.append(call)
    return calls
  if isinstance(payload, dict) and not payload:
    return []
  call = call_from_item(payload, numbering)
  return [call] if call is not None else []


def _is_wrapper(obj: Any) -> bool:
  """An object whose only job is to carry `.action` (an `Action`, or a look-alike that is not itself a call)."""
  if isinstance(obj, agent_types.Action):
    return True
  if isinstance(obj, (ToolCall, dict)) or not hasattr(obj, "action"):
    return False
  return not any(hasattr(obj, alias) for alias in NAME_ALIASES)


def extract_tool_calls(action: Any) -> Optional[List[ToolCall]]:
  """The tool calls an action amounts to, or None when it is not a tool-calling action."""
  payload = action
  while payload is not None and _is_wrapper(payload):
    payload = payload.action
  return calls_from_payload(payload) or None
