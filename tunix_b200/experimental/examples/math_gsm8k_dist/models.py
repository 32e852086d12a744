"""Model and tokenizer construction shared by the three worker nodes
(tunix/experimental/examples/math_gsm8k_dist/models.py).

Every node builds the same architecture from the same `--model` and `--seed`, so the trainer's and the rollout
worker's parameter manifests agree before the first weight sync. "tiny" is a two-layer model over a character
tokenizer that runs on a CPU in seconds; any other name is a preset of the model registry (e.g. "qwen3-0.6b",
"llama3.2-1b"), with random weights unless `--weights` names a local safetensors directory, and then `--tokenizer`
must name a local Hugging Face tokenizer directory.
"""
from __future__ import annotations

from typing import Any, Optional, Tuple

import torch

from ...common import test_utils

TINY_VOCAB = 160                      # the character tokenizer's ids for ASCII end at 130


def build_model(name: str = "tiny", seed: int = 0, weights: Optional[str] = None, device: Optional[str] = None,
                dtype: Optional[torch.dtype] = None) -> torch.nn.Module:
  from tunix_b200.models.transformer import ModelConfig, Transformer
  if name == "tiny":
    cfg = ModelConfig(num_layers=2, vocab_size=TINY_VOCAB, embed_dim=32, hidden_dim=64, num_heads=4, head_dim=8,
                      num_kv_heads=2)
    model = Transformer(cfg).init_weights(seed=seed, scale=0.3)
  else:
    from tunix_b200.models import automodel
    device = device or ("cuda" if torch.cuda.is_available() else "cpu")
    dtype = dtype or (torch.bfloat16 if device == "cuda" else torch.float32)
    if weights:
      return automodel.create_model_from_safe_tensors(name, weights, dtype=dtype, device=device)
    model = Transformer(automodel.call_model_config(name)).init_weights(seed=seed)
  device = device or ("cuda" if torch.cuda.is_available() else "cpu")
  if dtype is None and device == "cuda" and name != "tiny":
    dtype = torch.bfloat16
  return model.to(device=device, dtype=dtype) if dtype is not None else model.to(device)


def build_tokenizer(name: str = "tiny", tokenizer_path: Optional[str] = None) -> Any:
  if name == "tiny" and not tokenizer_path:
    return test_utils.MockTokenizer()
  if not tokenizer_path:
    raise ValueError(f"--tokenizer must name a local tokenizer directory for model {name!r}")
  from tunix_b200.generate import tokenizer_adapter
  return tokenizer_adapter.Tokenizer(tokenizer_type="huggingface", tokenizer_path=tokenizer_path)


def pad_and_eos(tokenizer: Any) -> Tuple[int, int]:
  pad, eos = tokenizer.pad_id(), tokenizer.eos_id()
  return int(pad if pad is not None else 0), int(eos)
