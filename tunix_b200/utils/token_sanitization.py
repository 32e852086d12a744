"""Removal of chat-control tokens from text that did not come from the template itself, so that
user or tool content cannot forge turn boundaries (tunix/utils/token_sanitization.py:19-86).
Removal repeats until a fixed point: a token split around another token re-forms after one
pass and must go too."""
from __future__ import annotations

import re
from typing import Iterable, Optional

_DEFAULT = ("<start_of_turn>", "<end_of_turn>", "<bos>", "<eos>", "<|begin_of_text|>", "<|end_of_text|>",
            "<|start_header_id|>", "<|end_header_id|>", "<|eot_id|>", "<|im_start|>", "<|im_end|>")
_DEFAULT_RE = re.compile("|".join(re.escape(t) for t in _DEFAULT))


def _to_text(content) -> str:
  if isinstance(content, str) or content is None:
    return content
  if isinstance(content, memoryview):
    content = content.tobytes()
  if isinstance(content, (bytes, bytearray)):
    return bytes(content).decode("utf-8", errors="replace")
  return str(content)


def sanitize_control_tokens(content, extra_tokens: Optional[Iterable[str]] = None, include_default: bool = True):
  text = _to_text(content)
  if not text:
    return text
  if include_default and not extra_tokens:
    rx = _DEFAULT_RE
  else:
    toks = set(_DEFAULT) if include_default else set()
    toks.update(t for t in (extra_tokens or ()) if t)
    if not toks:
      return text
    rx = re.compile("|".join(re.escape(t) for t in sorted(toks, key=lambda t: (-len(t), t))))
  while True:
    new = rx.sub("", text)
    if new == text:
      return new
    text = new
