"""Neutralises chat-control tokens inside user-provided text so that content cannot forge turn
boundaries (tunix/utils/token_sanitization.py)."""
from __future__ import annotations

import re

_CONTROL_PATTERNS = [
    r"<\|im_start\|>", r"<\|im_end\|>", r"<start_of_turn>", r"<end_of_turn>", r"<\|begin_of_text\|>",
    r"<\|end_of_text\|>", r"<\|start_header_id\|>", r"<\|end_header_id\|>", r"<\|eot_id\|>", r"<bos>", r"<eos>",
]
_RE = re.compile("|".join(_CONTROL_PATTERNS))


def sanitize_control_tokens(text):
  """Inserts a zero-width space after the opening bracket of every control token."""
  if not isinstance(text, str):
    return text
  return _RE.sub(lambda m: m.group(0)[0] + "​" + m.group(0)[1:], text)
