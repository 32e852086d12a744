"""Helpers of the agentic pipeline (tunix/rl/agentic/utils.py:26-274): padding, per-message
tokenisation with assistant masks, and the rollout / weight-sync lock."""
from __future__ import annotations

import asyncio
import contextlib
import threading
from typing import Any, Dict, List, Optional, Tuple

import numpy as np


def left_pad(x, length: int, pad, dtype=np.int32) -> np.ndarray:
  x = np.asarray(x, dtype=dtype)
  return x[-length:] if x.size >= length else np.concatenate([np.full(length - x.size, pad, dtype), x])


def right_pad(x, length: int, pad, dtype=np.int32) -> np.ndarray:
  x = np.asarray(x, dtype=dtype)
  return x[:length] if x.size >= length else np.concatenate([x, np.full(length - x.size, pad, dtype)])


def pad_prompt_and_completion(prompt_tokens, completion_tokens, max_prompt_length: int, max_generation_steps: int,
                              pad_id: int) -> Tuple[np.ndarray, np.ndarray, np.ndarray]:
  p = left_pad(prompt_tokens, max_prompt_length, pad_id)
  c = right_pad(completion_tokens, max_generation_steps, pad_id)
  return p, c, np.concatenate([p, c])


def get_recent_assistant_user_messages(messages: List[Dict[str, Any]]):
  """-> (last assistant message or None, the user/tool messages after it in order)."""
  env, assistant = [], None
  for m in reversed(messages):
    role = m.get("role")
    if role == "assistant":
      assistant = m
      break
    if role in ("user", "tool"):
      env.append(m)
  return assistant, env[::-1]


def convert_messages_to_string(message: Dict[str, Any]) -> Dict[str, str]:
  out = {}
  for k, v in message.items():
    if isinstance(v, np.ndarray):
      v = v.item()
    elif k == "content" and v is None:
      v = ""
    if not isinstance(v, str):
      raise ValueError(f"Message field {k} must be a string after preprocessing, got {type(v)}.")
    out[k] = v
  return out


def _encode(tokenizer, text: str) -> List[int]:
  try:
    return list(tokenizer.encode(text, add_special_tokens=False))
  except TypeError:
    return list(tokenizer.encode(text))


def convert_single_message(msg: Dict[str, str], tokenizer: Any, parser: Any, is_first: bool = False,
                           is_generation: bool = False) -> Tuple[List[int], List[int]]:
  """One message -> (token ids, mask); the mask is 1 on assistant messages only."""
  text = parser.parse(messages=[convert_messages_to_string(msg)], add_generation_prompt=is_generation,
                      is_first_msg=is_first)
  if msg["role"] == "assistant" and hasattr(parser, "assistant_token"):
    if text.startswith(parser.assistant_token):
      text = text[len(parser.assistant_token):]
  toks = _encode(tokenizer, text)
  return toks, [1 if msg["role"] == "assistant" else 0] * len(toks)


def tokenize_and_generate_masks(messages: List[Dict[str, str]], tokenizer: Any, parser: Any,
                                contains_first_msg: bool = False, contains_generation_msg: bool = False
                                ) -> Tuple[List[int], List[int]]:
  if hasattr(parser, "preprocess_messages"):
    messages = parser.preprocess_messages(messages)
  toks: List[int] = []
  masks: List[int] = []
  for i, m in enumerate(messages):
    t, k = convert_single_message(m, tokenizer, parser, contains_first_msg and i == 0,
                                  contains_generation_msg and i == len(messages) - 1)
    toks += t
    masks += k
  if hasattr(tokenizer, "dedup_bos_ids"):
    deduped = list(tokenizer.dedup_bos_ids(toks))
    if len(deduped) != len(toks):
      masks = masks[len(toks) - len(deduped):]
    toks = deduped
  return toks, masks


class RolloutSyncLock:
  """Many concurrent rollouts or one exclusive weight sync. A waiting sync blocks new rollouts,
  so a steady stream of episodes cannot starve the trainer."""

  def __init__(self):
    self._cv = threading.Condition()
    self._rollouts = 0
    self._syncing = False
    self._sync_waiting = 0

  def acquire_rollout(self) -> None:
    with self._cv:
      self._cv.wait_for(lambda: not self._syncing and self._sync_waiting == 0)
      self._rollouts += 1

  def release_rollout(self) -> None:
    with self._cv:
      self._rollouts -= 1
      if self._rollouts == 0:
        self._cv.notify_all()

  def acquire_weight_sync(self) -> None:
    with self._cv:
      self._sync_waiting += 1
      try:
        self._cv.wait_for(lambda: self._rollouts == 0 and not self._syncing)
      finally:
        self._sync_waiting -= 1
      self._syncing = True

  def release_weight_sync(self) -> None:
    with self._cv:
      self._syncing = False
      self._cv.notify_all()

  @contextlib.contextmanager
  def rollout(self):
    self.acquire_rollout()
    try:
      yield
    finally:
      self.release_rollout()

  @contextlib.contextmanager
  def weight_sync(self):
    self.acquire_weight_sync()
    try:
      yield
    finally:
      self.release_weight_sync()


def get_or_create_loop() -> asyncio.AbstractEventLoop:
  try:
    return asyncio.get_event_loop()
  except RuntimeError:
    loop = asyncio.new_event_loop()
    asyncio.set_event_loop(loop)
    return loop
