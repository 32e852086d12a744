"""Incremental chat-template rendering (tunix/rl/agentic/parser/chat_template_parser/parser.py:30-411).

A multi-turn episode is tokenised message by message, so each parser must render one message
such that the concatenation of the pieces equals the template applied to the whole
conversation: `parse(msgs, is_first_msg=True)` emits the conversation prefix (BOS, default
system prompt), later calls start with the message separator that the previous turn's
end-of-turn token did not emit. Message content is stripped of the template's own control
tokens first.
"""
from __future__ import annotations

import abc
import dataclasses
from typing import Dict, List, Tuple

import numpy as np

from .....utils import token_sanitization


@dataclasses.dataclass
class TokenConfig:
  bos_token: str = ""
  eos_token: str = ""
  eot_token: str = ""
  system_token: str = ""
  user_token: str = ""
  assistant_token: str = ""
  tool_start_token: str = ""
  tool_end_token: str = ""
  tool_response_start_token: str = ""
  tool_response_end_token: str = ""
  message_separator: str = ""


class BaseChatTemplateParser(abc.ABC):
  def __init__(self, tokenizer, enable_thinking: bool = True):
    self.tokenizer = tokenizer
    self.enable_thinking = enable_thinking
    self.tokens = self._init_tokens()
    self.generation_prompt = self._init_generation_prompt()
    self._tokens_to_sanitize = {v for k, v in dataclasses.asdict(self.tokens).items()
                                if k != "message_separator" and isinstance(v, str) and v}

  @abc.abstractmethod
  def _init_tokens(self) -> TokenConfig: ...

  @abc.abstractmethod
  def _init_generation_prompt(self) -> str: ...

  def parse(self, messages: List[Dict[str, str]], add_generation_prompt: bool = False,
            is_first_msg: bool = False) -> str:
    parts = []
    if is_first_msg:
      head = self._handle_first_message(messages)
      if head:
        parts.append(head)
    parts += [self._parse_message(m) for m in messages]
    if add_generation_prompt:
      parts.append(self.generation_prompt)
    sep = self.tokens.message_separator
    out = sep.join(parts)
    return sep + out if (not is_first_msg and out) else out

  def _handle_first_message(self, messages: List[Dict[str, str]]) -> str:
    return self.tokens.bos_token

  def _parse_message(self, message: Dict[str, str]) -> str:
    content = token_sanitization.sanitize_control_tokens(
        message["content"], extra_tokens=self._tokens_to_sanitize, include_default=not self._tokens_to_sanitize)
    render = {"system": self._parse_system, "user": self._parse_user, "assistant": self._parse_assistant,
              "tool": self._parse_tool}.get(message["role"])
    if render is None:
      raise NotImplementedError(f"Unsupported message role: {message['role']}")
    return render(content)

  def _parse_system(self, content: str) -> str:
    return self.tokens.system_token + content + self.tokens.eot_token

  def _parse_user(self, content: str) -> str:
    return self.tokens.user_token + content + self.tokens.eot_token

  def _parse_assistant(self, content: str) -> str:
    return self.tokens.assistant_token + content + self.tokens.eot_token

  def _parse_tool(self, content: str) -> str:
    t = self.tokens
    return t.user_token + t.tool_response_start_token + content + t.tool_response_end_token + t.eot_token

  @property
  def newline_tokens(self) -> List[int]:
    return []

  def update_assistant_end_tokens(self, tokens: np.ndarray) -> Tuple[np.ndarray, int]:
    """Tokens the template puts after an assistant turn that the model itself does not emit."""
    return tokens, 0


class DefaultChatTemplateParser(BaseChatTemplateParser):
  """Defers to the tokenizer's own `apply_chat_template`."""

  def _init_tokens(self) -> TokenConfig:
    return TokenConfig()

  def _init_generation_prompt(self) -> str:
    return ""

  def parse(self, messages, add_generation_prompt: bool = False, is_first_msg: bool = False) -> str:
    return self.tokenizer.apply_chat_template(messages, tokenize=False, add_generation_prompt=add_generation_prompt)


class QwenChatTemplateParser(BaseChatTemplateParser):
  def _init_tokens(self) -> TokenConfig:
    assistant = "<|im_start|>assistant\n" + ("" if self.enable_thinking else "<think>\n\n</think>\n\n")
    return TokenConfig(
        bos_token=getattr(self.tokenizer, "bos_token", "") or "", eos_token=getattr(self.tokenizer, "eos_token", "") or "",
        eot_token="<|im_end|>", system_token="<|im_start|>system\n", user_token="<|im_start|>user\n",
        assistant_token=assistant, tool_start_token="\n<tool_call>\n", tool_end_token="\n</tool_call>",
        tool_response_start_token="<tool_response>\n", tool_response_end_token="\n</tool_response>",
        message_separator="\n")

  def _init_generation_prompt(self) -> str:
    return self.tokens.assistant_token

  def _handle_first_message(self, messages) -> str:
    if messages[0]["role"] != "system":
      return self._parse_system("You are Qwen, created by Alibaba Cloud. You are a helpful assistant.")
    return ""


class LlamaChatTemplateParser(BaseChatTemplateParser):
  def _init_tokens(self) -> TokenConfig:
    hdr = lambda role: f"<|start_header_id|>{role}<|end_header_id|>\n\n"
    return TokenConfig(bos_token="<|begin_of_text|>", eot_token="<|eot_id|>", system_token=hdr("system"),
                       user_token=hdr("user"), assistant_token=hdr("assistant"), tool_start_token=hdr("tool"),
                       tool_end_token="<|eot_id|>", tool_response_start_token=hdr("tool_response"),
                       tool_response_end_token="<|eot_id|>")

  def _init_generation_prompt(self) -> str:
    return self.tokens.assistant_token


class GemmaChatTemplateParser(BaseChatTemplateParser):
  """Gemma has no system role: a leading system message is merged into the first user turn."""

  def _init_tokens(self) -> TokenConfig:
    return TokenConfig(bos_token="<bos>", eot_token="<end_of_turn>\n", user_token="<start_of_turn>user\n",
                       assistant_token="<start_of_turn>model\n")

  def _init_generation_prompt(self) -> str:
    return self.tokens.assistant_token

  def _parse_assistant(self, content: str) -> str:
    return self.tokens.assistant_token + content

  def _parse_system(self, content: str) -> str:
    raise ValueError("Gemma models do not support system messages directly. The system prompt should be the first "
                     "message and is handled by merging with the first user message.")

  def preprocess_messages(self, messages: List[Dict[str, str]]) -> List[Dict[str, str]]:
    msgs = [dict(m) for m in messages]
    if msgs and msgs[0]["role"] == "system":
      system = msgs.pop(0)
      if msgs and msgs[0]["role"] == "user":
        msgs[0]["content"] = system["content"] + "\n" + msgs[0]["content"]
      else:
        msgs.insert(0, {"role": "user", "content": system["content"]})
    return msgs

  def parse(self, messages, add_generation_prompt: bool = False, is_first_msg: bool = False) -> str:
    out = "".join(self._parse_message(m) for m in self.preprocess_messages(messages))
    return out + (self.generation_prompt if add_generation_prompt else "")


class Gemma4ChatTemplateParser(BaseChatTemplateParser):
  def __init__(self, tokenizer, enable_thinking: bool = True):
    super().__init__(tokenizer, enable_thinking=enable_thinking)
    self._tokens_to_sanitize.add("<turn|>")

  def _init_tokens(self) -> TokenConfig:
    return TokenConfig(
        bos_token="<bos>", eot_token="<turn|>\n",
        system_token="<|turn>system\n" + ("<|think|>" if self.enable_thinking else ""),
        user_token="<|turn>user\n",
        assistant_token="<|turn>model\n" + ("" if self.enable_thinking else "<|channel>thought\n<channel|>"),
        tool_start_token="<|tool_call>", tool_end_token="<tool_call|>", tool_response_start_token="<|tool_response>",
        tool_response_end_token="<tool_response|>", message_separator="")

  def _init_generation_prompt(self) -> str:
    return self.tokens.assistant_token

  def _handle_first_message(self, messages) -> str:
    head = self.tokens.bos_token
    if messages and messages[0]["role"] not in ("system", "developer") and self.enable_thinking:
      head += "<|turn>system\n<|think|><turn|>\n"
    return head

  def _parse_tool(self, content: str) -> str:
    return self.tokens.tool_response_start_token + content + self.tokens.tool_response_end_token

  def _parse_system(self, content: str) -> str:
    return self.tokens.system_token + content.strip() + self.tokens.eot_token

  def _parse_user(self, content: str) -> str:
    return self.tokens.user_token + content.strip() + self.tokens.eot_token

  def _parse_assistant(self, content: str) -> str:
    body = content.strip()
    prefix = "<|turn>model\n" if self.enable_thinking else self.tokens.assistant_token
    return prefix + body + ("\n" if body.endswith("<turn|>") else self.tokens.eot_token)

  @property
  def newline_tokens(self) -> List[int]:
    try:
      ids = self.tokenizer.encode("\n", add_special_tokens=False)
    except TypeError:
      ids = self.tokenizer.encode("\n")
    special = set()
    for attr in ("bos_id", "eos_id"):
      v = getattr(self.tokenizer, attr, None)
      v = v() if callable(v) else v
      if v is not None:
        special.add(v)
    return [t for t in ids if t not in special]

  def update_assistant_end_tokens(self, tokens: np.ndarray) -> Tuple[np.ndarray, int]:
    nl = self.newline_tokens
    return np.concatenate([tokens, np.asarray(nl, dtype=np.int32)], axis=0), len(nl)
