"""Helpers for tests written against this framework (tunix/tests/test_common.py:42-470).

Nothing here is a test itself. It gives tests small, fast, deterministic stand-ins:

  * `ToyTransformer(...)`: a real `Transformer` with toy dimensions (so every code path of the framework runs on it),
    `ToyTransformerWithScoreHead` for reward / value models, `get_lora_model`;
  * `MockVocab`: a word-level tokenizer over a fixed vocabulary with the sentencepiece method names next to the
    framework's own (`encode` / `decode` / `pad_id` ...), so it can stand in for either;
  * `assert_equal` / `assert_not_equal` / `assert_close` over nested dicts / lists / tuples of tensors and arrays
    (state dicts, optimizer states), reporting the path of the first leaf that differs;
  * `batch_templatize`, `validate_llm_outputs` for generation smoke tests; `delete_directory`;
    `free_device_memory` between heavy tests.
"""
from __future__ import annotations

import gc
import os
import shutil
from typing import Any, Dict, Iterable, Iterator, List, Mapping, Optional, Sequence, Tuple

import numpy as np
import torch

from ..models import lora as lora_lib
from ..models.transformer import ModelConfig, Transformer


# ---- tree comparisons ---------------------------------------------------------------------------------
def _as_array(leaf: Any) -> np.ndarray:
  if isinstance(leaf, torch.Tensor):
    return leaf.detach().float().cpu().numpy() if leaf.is_floating_point() else leaf.detach().cpu().numpy()
  return np.asarray(leaf)


def _leaves(tree: Any, path: str = "") -> Iterator[Tuple[str, Any]]:
  if isinstance(tree, torch.nn.Module):
    tree = dict(tree.state_dict())
  if isinstance(tree, Mapping):
    for key in sorted(tree, key=str):
      yield from _leaves(tree[key], f"{path}/{key}" if path else str(key))
  elif isinstance(tree, (list, tuple)):
    for index, item in enumerate(tree):
      yield from _leaves(item, f"{path}[{index}]")
  elif tree is not None:
    yield path, tree


def _paired(x: Any, y: Any) -> Iterator[Tuple[str, np.ndarray, np.ndarray]]:
  left, right = dict(_leaves(x)), dict(_leaves(y))
  if left.keys() != right.keys():
    only = sorted(set(left) ^ set(right))
    raise AssertionError(f"trees differ in structure; leaves on one side only: {only[:8]}")
  for path in left:
    yield path, _as_array(left[path]), _as_array(right[path])


def assert_equal(x: Any, y: Any, path: str = "") -> None:
  for leaf, a, b in _paired(x, y):
    np.testing.assert_array_equal(a, b, err_msg=f"leaf {path}{leaf}")


def assert_close(x: Any, y: Any, atol: float = 1e-5, rtol: float = 1e-5, path: str = "") -> None:
  for leaf, a, b in _paired(x, y):
    np.testing.assert_allclose(a, b, atol=atol, rtol=rtol, err_msg=f"leaf {path}{leaf}")


def assert_not_equal(x: Any, y: Any, path: str = "") -> None:
  """Every pair of leaves differs somewhere (what "the optimizer moved all of them" means)."""
  for leaf, a, b in _paired(x, y):
    if a.shape == b.shape and np.array_equal(a, b):
      raise AssertionError(f"leaf {path}{leaf} is equal on both sides")


# ---- toy models ------------------------------------------------------------------------------------------
def toy_config(vocab_size: int = 256, num_layers: int = 4, **overrides: Any) -> ModelConfig:
  base = dict(num_layers=num_layers, vocab_size=vocab_size, embed_dim=16, hidden_dim=32, num_heads=4, head_dim=4,
              num_kv_heads=2)
  base.update(overrides)
  return ModelConfig(**base)


def ToyTransformer(config: Optional[ModelConfig] = None, seed: int = 0, scale: float = 0.3, **overrides: Any
                   ) -> Transformer:  # noqa: N802 - the reference's name for it
  return Transformer(config or toy_config(**overrides)).init_weights(seed=seed, scale=scale)


class ToyTransformerWithScoreHead(torch.nn.Module):
  """A transformer whose output is one score per position: the final hidden states through a linear head. Call
  signature and return shape are those reward and value models have in this framework: `(ids, positions, cache,
  mask) -> ([B, T, 1], cache)`."""

  def __init__(self, transformer: Optional[Transformer] = None, seed: int = 0):
    super().__init__()
    self.transformer = transformer or ToyTransformer(seed=seed)
    generator = torch.Generator().manual_seed(seed + 1)
    width = self.transformer.config.embed_dim
    self.score = torch.nn.Parameter(torch.randn(width, 1, generator=generator) / width ** 0.5)

  @property
  def config(self) -> ModelConfig:
    return self.transformer.config

  def forward(self, ids, positions=None, cache=None, attention_mask=None, **kwargs):
    hidden, cache = self.transformer(ids, positions, cache, attention_mask, skip_lm_head=True, **kwargs)
    return hidden.to(self.score.dtype) @ self.score, cache


def get_lora_model(model: Optional[Transformer] = None, module_path: str = ".*(q_proj|v_proj|gate_proj|down_proj)",
                   rank: int = 4, alpha: float = 2.0, seed: int = 0, randomize_b: bool = True) -> Transformer:
  """Adapters on the matching projections. `randomize_b` fills the B factors (zero by construction) so that the
  adapters change the output, which is what a merge or export test needs."""
  model = lora_lib.apply_lora_to_model(model or ToyTransformer(seed=seed), rank=rank, alpha=alpha, module_path=module_path)
  if randomize_b:
    generator = torch.Generator().manual_seed(seed + 7)
    with torch.no_grad():
      for name, p in model.named_parameters():
        if getattr(p, "is_lora", False) and "lora_b" in name:
          p.copy_(torch.randn(p.shape, generator=generator).to(p.dtype) * 0.05)
  return model


def get_dummy_inputs_for_lora_toy_transformer_tests(batch: int = 2, length: int = 8, vocab_size: int = 256, seed: int = 0
                                                    ) -> Dict[str, torch.Tensor]:
  generator = torch.Generator().manual_seed(seed)
  ids = torch.randint(3, vocab_size, (batch, length), generator=generator)
  return {"input_tokens": ids, "positions": torch.arange(length).expand(batch, length),
          "attention_mask": torch.tril(torch.ones(length, length, dtype=torch.bool)).expand(batch, length, length)}


# ---- tokenizer -----------------------------------------------------------------------------------------------
class MockVocab:
  """Word-level tokenizer over a fixed vocabulary; unknown words are dropped on encoding."""

  WORDS = ("<pad>", "<s>", "</s>", "input", "string", "hello", "world", "Hello", "there", "!", "My", "name", "is",
           "Morgane", "Tunix", "Parallax", "PT", "library", "distributed", "training", "optimizer", "quantization")
  IMAGE_WORDS = ("<img>", "<soi>", "<eoi>", "<doubleline>")

  def __init__(self, mapping_text_to_id: Optional[Mapping[str, int]] = None, is_multimodal: bool = False):
    words = self.WORDS + (self.IMAGE_WORDS if is_multimodal else ())
    self._to_id: Dict[str, int] = dict(mapping_text_to_id) if mapping_text_to_id else {w: i for i, w in enumerate(words)}
    self._to_word = {i: w for w, i in self._to_id.items()}

  def pad_id(self) -> int:
    return 0

  def bos_id(self) -> int:
    return 1

  def eos_id(self) -> int:
    return 2

  def vocab_size(self) -> int:
    return len(self._to_id)

  def encode(self, text: str, **kwargs: Any) -> List[int]:
    return [self._to_id[w] for w in text.split(" ") if w in self._to_id]

  def decode(self, ids: Iterable[int], **kwargs: Any) -> str:
    return " ".join(self._to_word[int(i)] for i in ids)

  # the sentencepiece spellings of the same three
  GetPieceSize = vocab_size          # noqa: N815
  EncodeAsIds = encode               # noqa: N815
  DecodeIds = decode                 # noqa: N815


# ---- generation smoke tests --------------------------------------------------------------------------------
def batch_templatize(prompts: Sequence[str], tokenizer: Any) -> List[str]:
  if not hasattr(tokenizer, "apply_chat_template"):
    raise TypeError(f"{type(tokenizer).__name__} has no apply_chat_template")
  return [tokenizer.apply_chat_template([{"role": "user", "content": p}], tokenize=False, add_generation_prompt=True)
          for p in prompts]


def validate_llm_outputs(expected_output_pattern: Sequence[Tuple[str, Sequence[str]]], serving_outputs: Sequence[str]) -> None:
  if len(expected_output_pattern) != len(serving_outputs):
    raise AssertionError(f"{len(expected_output_pattern)} expectations for {len(serving_outputs)} outputs")
  for (prompt, keywords), generated in zip(expected_output_pattern, serving_outputs):
    missing = [k for k in keywords if k.lower() not in generated.strip().lower()]
    if missing:
      raise AssertionError(f"Response {generated!r} for prompt {prompt!r} does not contain expected keyword(s) {missing}.")


# ---- housekeeping ----------------------------------------------------------------------------------------------
def delete_directory(path: str) -> None:
  if os.path.isdir(path):
    shutil.rmtree(path)
  elif os.path.exists(path):
    raise NotADirectoryError(path)


def free_device_memory() -> None:
  """Drops unreferenced tensors and returns cached blocks to the driver (between heavy tests on one GPU)."""
  gc.collect()
  if torch.cuda.is_available():
    torch.cuda.empty_cache()
