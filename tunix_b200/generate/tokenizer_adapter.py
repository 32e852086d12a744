"""One interface over SentencePiece, Hugging Face and duck-typed tokenizers
(tunix/generate/tokenizer_adapter.py:28-307): `encode / decode / bos_id / eos_id / pad_id`, `dedup_bos_ids`,
`apply_chat_template` (Gemma turn format where the tokenizer has no template of its own).

The adapter does not branch on the tokenizer's kind in every method. Construction picks one *backend* - a small
object that knows how its kind spells each operation - and every call is forwarded to it:

  `_SentencePiece`  ids through `EncodeAsIds` / `DecodeIds`; an undefined pad id (-1) is an error
  `_HuggingFace`    ids through `encode` / `decode`, special ids are attributes; a missing pad token becomes the
                    end-of-sequence token; chat formatting by the tokenizer's own template
  `_Duck`           any object with the five methods; its `apply_chat_template` is used if it has one
"""
from __future__ import annotations

import enum
from typing import Any, Dict, List, Optional, Sequence, Union

import numpy as np

from ..utils import token_sanitization

try:
  import sentencepiece as spm
except Exception:  # pragma: no cover
  spm = None

_REQUIRED = ("encode", "decode", "bos_id", "eos_id", "pad_id")
_HF_BASE = "tokenization_utils_base.PreTrainedTokenizerBase"


class TokenizerType(enum.Enum):
  SP = "sp"
  HF = "hf"
  NONE = "none"


def gemma_chat_text(messages: Sequence[Dict[str, str]], add_generation_prompt: bool) -> str:
  """Gemma's turn format; roles other than `user` and `model` are left out."""
  turns = [f"<start_of_turn>{m.get('role')}\n{m.get('content')}<end_of_turn>\n" for m in messages
           if m.get("role") in ("user", "model")]
  return "".join(turns) + ("<start_of_turn>model\n" if add_generation_prompt else "")


class _Duck:
  kind = TokenizerType.NONE

  def __init__(self, tok: Any):
    self.tok = tok

  @staticmethod
  def accepts(tok: Any) -> bool:
    return all(hasattr(tok, m) for m in _REQUIRED)

  def encode(self, text, **kw):
    return self.tok.encode(text, **kw)

  def decode(self, ids, **kw):
    return self.tok.decode(ids, **kw)

  def bos(self):
    return self.tok.bos_id()

  def eos(self):
    return self.tok.eos_id()

  def pad(self):
    return self.tok.pad_id()

  def chat(self, messages, add_generation_prompt, tokenize, **kw):
    if hasattr(self.tok, "apply_chat_template"):
      return self.tok.apply_chat_template(messages, add_generation_prompt=add_generation_prompt, tokenize=tokenize, **kw)
    text = gemma_chat_text(messages, add_generation_prompt)
    return self.encode(text) if tokenize else text


class _SentencePiece(_Duck):
  kind = TokenizerType.SP

  @staticmethod
  def accepts(tok: Any) -> bool:
    return spm is not None and isinstance(tok, spm.SentencePieceProcessor)

  def encode(self, text, **kw):
    return self.tok.EncodeAsIds(text, **kw)

  def decode(self, ids, **kw):
    return self.tok.DecodeIds(ids, **kw)

  def pad(self):
    pad = self.tok.pad_id()
    if pad == -1:
      raise ValueError("SentencePiece tokenizer has a undefined pad_id.")
    return pad

  def chat(self, messages, add_generation_prompt, tokenize, **kw):
    text = gemma_chat_text(messages, add_generation_prompt)
    return self.encode(text) if tokenize else text


class _HuggingFace(_Duck):
  kind = TokenizerType.HF

  @staticmethod
  def accepts(tok: Any) -> bool:
    return any(f"{c.__module__}.{c.__name__}".endswith(_HF_BASE) for c in type(tok).__mro__)

  def bos(self):
    return self.tok.bos_token_id

  def eos(self):
    return self.tok.eos_token_id

  def pad(self):
    if self.tok.pad_token_id is None:
      self.tok.pad_token = self.tok.eos_token
    return self.tok.pad_token_id

  def chat(self, messages, add_generation_prompt, tokenize, **kw):
    return self.tok.apply_chat_template(messages, add_generation_prompt=add_generation_prompt, tokenize=tokenize, **kw)


_BACKENDS = (_SentencePiece, _HuggingFace, _Duck)      # most specific first


class TokenizerAdapter:

  def __init__(self, tokenizer: Any):
    self._tokenizer = tokenizer
    backend = next((b for b in _BACKENDS if b.accepts(tokenizer)), None)
    if backend is None:
      missing = [m for m in _REQUIRED if not hasattr(tokenizer, m)]
      raise ValueError("Your tokenizer should either be a `spm.SentencePieceProcessor` tokenizer, a HuggingFace "
                       "tokenizer, or it should have the following methods: "
                       '`["encode", "decode", "bos_id", "eos_id", "pad_id"]`. Received: '
                       f"`type(tokenizer)` = {type(tokenizer)}, with missing methods: {missing}.")
    self._tokenizer_backend = backend(tokenizer)
    self._tokenizer_type = backend.kind

  @property
  def tokenizer(self) -> Any:
    return self._tokenizer

  def __getattr__(self, name: str) -> Any:
    if name.startswith("_tokenizer"):          # not set yet (unpickling, failed construction): no recursion
      raise AttributeError(name)
    return getattr(self._tokenizer, name)

  def encode(self, text: str, **kwargs) -> List[int]:
    return self._tokenizer_backend.encode(text, **kwargs)

  def decode(self, ids: List[int], **kwargs) -> str:
    return self._tokenizer_backend.decode(ids, **kwargs)

  def bos_id(self) -> int:
    return self._tokenizer_backend.bos()

  def eos_id(self) -> int:
    return self._tokenizer_backend.eos()

  def pad_id(self) -> int:
    return self._tokenizer_backend.pad()

  def dedup_bos_ids(self, ids: List[int]) -> List[int]:
    """Collapses a run of beginning-of-sequence tokens at the start into one."""
    bos, first = self.bos_id(), 0
    while first + 1 < len(ids) and ids[first] == bos and ids[first + 1] == bos:
      first += 1
    return ids[first:]

  def apply_chat_template(self, messages: List[Dict[str, str]], add_generation_prompt: bool = True,
                          tokenize: bool = False, **kwargs) -> Union[str, List[int]]:
    """Control-token look-alikes in message contents are neutralised before formatting."""
    clean = [{**m, "content": token_sanitization.sanitize_control_tokens(m["content"])} for m in messages]
    return self._tokenizer_backend.chat(clean, add_generation_prompt, tokenize, **kwargs)

  def _apply_gemma_chat_template(self, messages, add_generation_prompt: bool, tokenize: bool):
    text = gemma_chat_text(messages, add_generation_prompt)
    return self.encode(text) if tokenize else text


def _load_sentencepiece(path: str, add_bos: Optional[bool], add_eos: Optional[bool]):
  if spm is None:
    raise ImportError("sentencepiece is not installed")
  tok = spm.SentencePieceProcessor()
  with open(path, "rb") as f:
    tok.LoadFromSerializedProto(f.read())
  extras = ":".join(flag for flag, on in (("bos", add_bos), ("eos", add_eos)) if on)
  if extras:
    tok.SetEncodeExtraOptions(extras)
  return tok


class Tokenizer(TokenizerAdapter):
  """Loads a tokenizer from a local path: `tokenizer_type` "huggingface" or "sentencepiece"."""

  def __init__(self, tokenizer_type: str = "sentencepiece", tokenizer_path: str = "", add_bos: Optional[bool] = True,
               add_eos: Optional[bool] = True, hf_access_token: Optional[str] = None):
    self.tokenizer_type = tokenizer_type
    if tokenizer_type == "huggingface":
      import transformers
      loaded = transformers.AutoTokenizer.from_pretrained(tokenizer_path, add_bos_token=add_bos, add_eos_token=add_eos,
                                                          token=hf_access_token)
    elif tokenizer_type == "sentencepiece":
      loaded = _load_sentencepiece(tokenizer_path, add_bos, add_eos)
    else:
      raise ValueError(f"Unsupported tokenizer_type: {tokenizer_type}")
    super().__init__(loaded)

  def tokenize(self, example: str, prefix: str = "", suffix: str = "", add_eos: bool = True) -> np.ndarray:
    """[bos] prefix+example+suffix [eos] as int32; the text is sanitised and encoded without the tokenizer's own
    special tokens."""
    text = prefix + token_sanitization.sanitize_control_tokens(example) + suffix
    body = (self.encode(text, add_special_tokens=False) if self.tokenizer_type == "huggingface"
            else self.tokenizer.EncodeAsIds(text))
    ids = ([self.bos_id()] if self.bos_id() else []) + list(body) + ([self.eos_id()] if add_eos else [])
    return np.array(ids, dtype=np.int32)
