"""Incremental chat-template rendering (tunix/rl/agentic/parser/chat_template_parser/parser.py:30-411).

A multi-turn episode is tokenised message by message, so a parser must render one message such that the
concatenation of the pieces equals the template applied to the whole conversation: `parse(msgs,
is_first_msg=True)` emits the conversation preamble (BOS, default system prompt), later calls start with the
separator that the previous turn's end-of-turn token did not emit. Message content is stripped of the
template's own control tokens first.

A template is data plus a few hooks. The data is `TokenConfig`; from it `frames()` derives, per role, the text
that opens and closes a turn. The one renderer (`BaseChatTemplateParser.parse`) is
`preamble + separator.join(open + content + close for each message) + generation prompt`; model families
override `frames()`, `preamble()`, `normalise()` (message list rewriting, e.g. Gemma's missing system role) or
`body()` (content clean-up) where their template deviates.
"""
from __future__ import annotations

import abc
import dataclasses
from typing import Dict, List, Sequence, Tuple

import numpy as np

from .....utils import token_sanitization

Message = Dict[str, str]
Frame = Tuple[str, str]            # (text before the content, text after it)


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

  def control_tokens(self) -> set:
    return {v for k, v in dataclasses.asdict(self).items() if k != "message_separator" and isinstance(v, str) and v}


class BaseChatTemplateParser(abc.ABC):

  def __init__(self, tokenizer, enable_thinking: bool = True):
    self.tokenizer = tokenizer
    self.enable_thinking = enable_thinking
    self.tokens = self._init_tokens()
    self.generation_prompt = self._init_generation_prompt()
    self._tokens_to_sanitize = self.tokens.control_tokens()
    self._frames = self.frames()

  # ---- what a family defines
  @abc.abstractmethod
  def _init_tokens(self) -> TokenConfig: ...

  def _init_generation_prompt(self) -> str:
    return self.tokens.assistant_token

  def frames(self) -> Dict[str, Frame]:
    """Opening and closing text of a turn, per role. A tool result is a user turn wrapping the response markers."""
    t = self.tokens
    return {"system": (t.system_token, t.eot_token), "user": (t.user_token, t.eot_token),
            "assistant": (t.assistant_token, t.eot_token),
            "tool": (t.user_token + t.tool_response_start_token, t.tool_response_end_token + t.eot_token)}

  def preamble(self, messages: Sequence[Message]) -> str:
    """Text in front of the first message of a conversation."""
    return self.tokens.bos_token

  def normalise(self, messages: Sequence[Message]) -> Sequence[Message]:
    return messages

  def body(self, role: str, content: str) -> str:
    return content

  # ---- the renderer
  def _clean(self, content: str) -> str:
    return token_sanitization.sanitize_control_tokens(content, extra_tokens=self._tokens_to_sanitize,
                                                      include_default=not self._tokens_to_sanitize)

  def _parse_message(self, message: Message) -> str:
    role = message["role"]
    if role not in self._frames:
      raise NotImplementedError(f"Unsupported message role: {role}")
    return self.render_turn(role, self.body(role, self._clean(message["content"])))

  def render_turn(self, role: str, content: str) -> str:
    before, after = self._frames[role]
    return before + content + after

  def parse(self, messages: List[Message], add_generation_prompt: bool = False, is_first_msg: bool = False) -> str:
    pieces = [self._parse_message(m) for m in self.normalise(messages)]
    if is_first_msg:
      head = self.preamble(messages)
      if head:
        pieces.insert(0, head)
    if add_generation_prompt:
      pieces.append(self.generation_prompt)
    sep = self.tokens.message_separator
    text = sep.join(pieces)
    return text if (is_first_msg or not text) else sep + text

  # ---- what follows an assistant turn
  @property
  def newline_tokens(self) -> List[int]:
    return []

  def update_assistant_end_tokens(self, tokens: np.ndarray) -> Tuple[np.ndarray, int]:
    """Tokens the template puts after an assistant turn that the model itself does not emit: (tokens with them
    appended, how many were appended)."""
    extra = self.newline_tokens
    if not extra:
      return tokens, 0
    return np.concatenate([tokens, np.asarray(extra, dtype=np.int32)], axis=0), len(extra)


class DefaultChatTemplateParser(BaseChatTemplateParser):
  """Defers to the tokenizer's own `apply_chat_template`."""

  def _init_tokens(self) -> TokenConfig:
    return TokenConfig()

  def parse(self, messages, add_generation_prompt: bool = False, is_first_msg: bool = False) -> str:
    return self.tokenizer.apply_chat_template(messages, tokenize=False, add_generation_prompt=add_generation_prompt)


class QwenChatTemplateParser(BaseChatTemplateParser):
  DEFAULT_SYSTEM = "You are Qwen, created by Alibaba Cloud. You are a helpful assistant."
  NO_THINKING = "<think>\n\n</think>\n\n"

  def _init_tokens(self) -> TokenConfig:
    special = lambda name: getattr(self.tokenizer, name, "") or ""
    return TokenConfig(
        bos_token=special("bos_token"), eos_token=special("eos_token"), eot_token="<|im_end|>",
        system_token="<|im_start|>system\n", user_token="<|im_start|>user\n",
        assistant_token="<|im_start|>assistant\n" + ("" if self.enable_thinking else self.NO_THINKING),
        tool_start_token="\n<tool_call>\n", tool_end_token="\n</tool_call>",
        tool_response_start_token="<tool_response>\n", tool_response_end_token="\n</tool_response>",
        message_separator="\n")

  def preamble(self, messages) -> str:
    """Qwen's template supplies a system prompt when the conversation has none (and prints no BOS)."""
    return "" if messages[0]["role"] == "system" else self.render_turn("system", self.DEFAULT_SYSTEM)


class LlamaChatTemplateParser(BaseChatTemplateParser):

  @staticmethod
  def _header(role: str) -> str:
    return f"<|start_header_id|>{role}<|end_header_id|>\n\n"

  def _init_tokens(self) -> TokenConfig:
    h = self._header
    return TokenConfig(bos_token="<|begin_of_text|>", eot_token="<|eot_id|>", system_token=h("system"),
                       user_token=h("user"), assistant_token=h("assistant"), tool_start_token=h("tool"),
                       tool_end_token="<|eot_id|>", tool_response_start_token=h("tool_response"),
                       tool_response_end_token="<|eot_id|>")


class GemmaChatTemplateParser(BaseChatTemplateParser):
  """Gemma has no system role: a leading system message is merged into the first user turn. Turns already end
  with a newline, there is no separator and no preamble, and an assistant turn is left open."""

  def _init_tokens(self) -> TokenConfig:
    return TokenConfig(bos_token="<bos>", eot_token="<end_of_turn>\n", user_token="<start_of_turn>user\n",
                       assistant_token="<start_of_turn>model\n")

  def frames(self) -> Dict[str, Frame]:
    out = super().frames()
    out["assistant"] = (self.tokens.assistant_token, "")
    return out

  def render_turn(self, role: str, content: str) -> str:
    if role == "system":
      raise ValueError("Gemma models do not support system messages directly. The system prompt should be the first "
                       "message and is handled by merging with the first user message.")
    return super().render_turn(role, content)

  def preprocess_messages(self, messages: List[Message]) -> List[Message]:
    rest = [dict(m) for m in messages]
    if not rest or rest[0]["role"] != "system":
      return rest
    system = rest.pop(0)["content"]
    if rest and rest[0]["role"] == "user":
      rest[0]["content"] = system + "\n" + rest[0]["content"]
      return rest
    return [{"role": "user", "content": system}] + rest

  normalise = preprocess_messages

  def parse(self, messages, add_generation_prompt: bool = False, is_first_msg: bool = False) -> str:
    return super().parse(messages, add_generation_prompt=add_generation_prompt, is_first_msg=False)

  def preamble(self, messages) -> str:
    return ""


class Gemma4ChatTemplateParser(BaseChatTemplateParser):
  TURN_END = "<turn|>"
  THINK_SYSTEM = "<|turn>system\n<|think|><turn|>\n"

  def __init__(self, tokenizer, enable_thinking: bool = True):
    super().__init__(tokenizer, enable_thinking=enable_thinking)
    self._tokens_to_sanitize.add(self.TURN_END)

  def _init_tokens(self) -> TokenConfig:
    think = self.enable_thinking
    return TokenConfig(
        bos_token="<bos>", eot_token=self.TURN_END + "\n",
        system_token="<|turn>system\n" + ("<|think|>" if think else ""), user_token="<|turn>user\n",
        assistant_token="<|turn>model\n" + ("" if think else "<|channel>thought\n<channel|>"),
        tool_start_token="<|tool_call>", tool_end_token="<tool_call|>", tool_response_start_token="<|tool_response>",
        tool_response_end_token="<tool_response|>", message_separator="")

  def frames(self) -> Dict[str, Frame]:
    out = super().frames()
    t = self.tokens
    out["tool"] = (t.tool_response_start_token, t.tool_response_end_token)     # tool results are bare, not user turns
    return out

  def preamble(self, messages) -> str:
    """With thinking on, a conversation without a system turn gets one that only switches thinking on."""
    needs_switch = self.enable_thinking and messages and messages[0]["role"] not in ("system", "developer")
    return self.tokens.bos_token + (self.THINK_SYSTEM if needs_switch else "")

  def body(self, role: str, content: str) -> str:
    return content if role == "tool" else content.strip()

  def render_turn(self, role: str, content: str) -> str:
    if role != "assistant":
      return super().render_turn(role, content)
    # a past assistant turn is replayed without the empty-thought stub; one that already closed its turn gets
    # only the newline
    opener = "<|turn>model\n" if self.enable_thinking else self.tokens.assistant_token
    return opener + content + ("\n" if content.endswith(self.TURN_END) else self.tokens.eot_token)

  @property
  def newline_tokens(self) -> List[int]:
    try:
      ids = self.tokenizer.encode("\n", add_special_tokens=False)
    except TypeError:
      ids = self.tokenizer.encode("\n")
    special = set()
    for name in ("bos_id", "eos_id"):
      value = getattr(self.tokenizer, name, None)
      value = value() if callable(value) else value
      if value is not None:
        special.add(value)
    return [t for t in ids if t not in special]
