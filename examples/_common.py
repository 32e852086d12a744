"""Shared by the example scripts: a tiny model, a character tokenizer and the device choice."""
from __future__ import annotations

import torch

from tunix_b200.models.transformer import ModelConfig, Transformer


class CharTokenizer:
  """One id per character (0 pad, 1 bos, 2 eos)."""

  def __init__(self, vocab_size: int = 160):
    self.vocab_size = vocab_size

  def encode(self, text, **_):
    return [3 + ord(c) % (self.vocab_size - 3) for c in text]

  def decode(self, ids, **_):
    return "".join(chr(int(i) - 3) for i in ids if int(i) >= 3)

  def bos_id(self):
    return 1

  def eos_id(self):
    return 2

  def pad_id(self):
    return 0


def tiny(layers: int = 2, width: int = 64, vocab: int = 160, seed: int = 0, scale: float = 0.1) -> Transformer:
  cfg = ModelConfig(num_layers=layers, vocab_size=vocab, embed_dim=width, hidden_dim=2 * width, num_heads=4,
                    head_dim=width // 4, num_kv_heads=2)
  return Transformer(cfg).init_weights(seed=seed, scale=scale)


def device() -> torch.device:
  return torch.device("cuda") if torch.cuda.is_available() else torch.device("cpu")
