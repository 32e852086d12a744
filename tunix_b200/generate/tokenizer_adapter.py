"""One interface over SentencePiece, Hugging Face and duck-typed tokenizers
(tunix/generate/tokenizer_adapter.py:28-307): `encode/decode/bos_id/eos_id/pad_id`,
`dedup_bos_ids`, `apply_chat_template` (Gemma turn format as the fallback)."""
from __future__ import annotations

import enum
import inspect
from typing import Any, Dict, List, Optional, Union

import numpy as np

from ..utils import token_sanitization

try:
  import sentencepiece as spm
except Exception:  # pragma: no cover
  spm = None


class TokenizerType(enum.Enum):
  SP = "sp"
  HF = "hf"
  NONE = "none"


class TokenizerAdapter:

  def __init__(self, tokenizer: Any):
    self._tokenizer = tokenizer
    missing = self._missing_methods()
    if spm is not None and isinstance(tokenizer, spm.SentencePieceProcessor):
      self._tokenizer_type = TokenizerType.SP
    elif self._is_hf_tokenizer():
      self._tokenizer_type = TokenizerType.HF
    elif not missing:
      self._tokenizer_type = TokenizerType.NONE
    else:
      raise ValueError("Your tokenizer should either be a `spm.SentencePieceProcessor` tokenizer, a HuggingFace "
                       "tokenizer, or it should have the following methods: "
                       '`["encode", "decode", "bos_id", "eos_id", "pad_id"]`. Received: '
                       f"`type(tokenizer)` = {type(tokenizer)}, with missing methods: {missing}.")

  def encode(self, text: str, **kwargs) -> List[int]:
    if self._tokenizer_type == TokenizerType.SP:
      return self._tokenizer.EncodeAsIds(text, **kwargs)
    return self._tokenizer.encode(text, **kwargs)

  def decode(self, ids: List[int], **kwargs) -> str:
    if self._tokenizer_type == TokenizerType.SP:
      return self._tokenizer.DecodeIds(ids, **kwargs)
    return self._tokenizer.decode(ids, **kwargs)

  def bos_id(self) -> int:
    if self._tokenizer_type == TokenizerType.HF:
      return self._tokenizer.bos_token_id
    return self._tokenizer.bos_id()

  def eos_id(self) -> int:
    if self._tokenizer_type == TokenizerType.HF:
      return self._tokenizer.eos_token_id
    return self._tokenizer.eos_id()

  def pad_id(self) -> int:
    if self._tokenizer_type == TokenizerType.SP:
      r = self._tokenizer.pad_id()
      if r == -1:
        raise ValueError("SentencePiece tokenizer has a undefined pad_id.")
      return r
    if self._tokenizer_type == TokenizerType.HF:
      if self._tokenizer.pad_token_id is None:
        self._tokenizer.pad_token = self._tokenizer.eos_token
      return self._tokenizer.pad_token_id
    return self._tokenizer.pad_id()

  def dedup_bos_ids(self, ids: List[int]) -> List[int]:
    i = 0
    while i < len(ids) - 1 and ids[i] == ids[i + 1] == self.bos_id():
      i += 1
    return ids[i:]

  def _missing_methods(self) -> List[str]:
    return [m for m in ("encode", "decode", "bos_id", "eos_id", "pad_id") if not hasattr(self._tokenizer, m)]

  def _is_hf_tokenizer(self) -> bool:
    names = [c.__module__ + "." + c.__name__ for c in inspect.getmro(type(self._tokenizer))]
    return any(n.endswith("tokenization_utils_base.PreTrainedTokenizerBase") for n in names)

  @property
  def tokenizer(self) -> Any:
    return self._tokenizer

  def __getattr__(self, name: str) -> Any:
    if name.startswith("_tokenizer"):
      raise AttributeError(name)
    return getattr(self._tokenizer, name)

  def apply_chat_template(self, messages: List[Dict[str, str]], add_generation_prompt: bool = True,
                          tokenize: bool = False, **kwargs) -> Union[str, List[int]]:
    messages = [{**m, "content": token_sanitization.sanitize_control_tokens(m["content"])} for m in messages]
    if self._tokenizer_type == TokenizerType.HF or (
        self._tokenizer_type == TokenizerType.NONE and hasattr(self._tokenizer, "apply_chat_template")):
      return self._tokenizer.apply_chat_template(messages, add_generation_prompt=add_generation_prompt,
                                                 tokenize=tokenize, **kwargs)
    return self._apply_gemma_chat_template(messages, add_generation_prompt, tokenize)

  def _apply_gemma_chat_template(self, messages, add_generation_prompt: bool, tokenize: bool):
    chat = ""
    for m in messages:
      role, content = m.get("role"), m.get("content")
      if role in ("user", "model"):
        chat += f"<start_of_turn>{role}\n{content}<end_of_turn>\n"
    if add_generation_prompt:
      chat += "<start_of_turn>model\n"
    return self.encode(chat) if tokenize else chat


class Tokenizer(TokenizerAdapter):
  """Loads a tokenizer from a local path: `tokenizer_type` "huggingface" or "sentencepiece"."""

  def __init__(self, tokenizer_type: str = "sentencepiece", tokenizer_path: str = "", add_bos: Optional[bool] = True,
               add_eos: Optional[bool] = True, hf_access_token: Optional[str] = None):
    self.tokenizer_type = tokenizer_type
    if tokenizer_type == "huggingface":
      import transformers
      tok = transformers.AutoTokenizer.from_pretrained(tokenizer_path, add_bos_token=add_bos, add_eos_token=add_eos,
                                                       token=hf_access_token)
    elif tokenizer_type == "sentencepiece":
      if spm is None:
        raise ImportError("sentencepiece is not installed")
      with open(tokenizer_path, "rb") as f:
        proto = f.read()
      tok = spm.SentencePieceProcessor()
      tok.LoadFromSerializedProto(proto)
      opts = [o for o, on in (("bos", add_bos), ("eos", add_eos)) if on]
      if opts:
        tok.SetEncodeExtraOptions(":".join(opts))
    else:
      raise ValueError(f"Unsupported tokenizer_type: {tokenizer_type}")
    super().__init__(tok)

  def tokenize(self, example: str, prefix: str = "", suffix: str = "", add_eos: bool = True) -> np.ndarray:
    example = token_sanitization.sanitize_control_tokens(example)
    ids: List[int] = []
    if self.bos_id():
      ids.append(self.bos_id())
    if self.tokenizer_type == "huggingface":
      ids.extend(self.encode(prefix + example + suffix, add_special_tokens=False))
    else:
      ids.extend(self.tokenizer.EncodeAsIds(prefix + example + suffix))
    if add_eos:
      ids.append(self.eos_id())
    return np.array(ids, dtype=np.int32)
