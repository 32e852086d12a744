"""LoRA / QLoRA adapters.

`apply_lora_to_model(model, rank, alpha, module_path)` adds `(x A^T) B^T * alpha / rank` to every
projection whose dotted path matches the regular expression, which is what the reference gets
from its LoRA provider (tunix/cli/utils/model.py:31-77): paths look like
`layers.0.attn.q_proj`, `layers.3.mlp.down_proj`. Base weights are frozen. With
`weight_qtype="nf4"` the frozen base weights are also stored 4-bit (QLoRA).
"""
from __future__ import annotations

import re
from typing import List, Optional

import torch

from .transformer import Linear


def lora_targets(model: torch.nn.Module, module_path: str) -> List[tuple]:
  pat = re.compile(module_path)
  out = []
  for mod_name, mod in model.named_modules():
    if not isinstance(mod, Linear):
      continue
    parent = mod_name.rsplit(".", 1)[0] if "." in mod_name else ""
    for slice_name in mod.slices:
      logical = f"{parent}.{slice_name}" if slice_name else mod_name
      if pat.fullmatch(logical) or pat.search(logical) and pat.pattern.startswith(".*"):
        out.append((mod, slice_name, logical))
  return out


def apply_lora_to_model(model: torch.nn.Module, rank: int, alpha: float,
                        module_path: str = ".*(q_proj|k_proj|v_proj|o_proj|gate_proj|up_proj|down_proj)",
                        weight_qtype: Optional[str] = None, tile_size: int = 64, dtype=None) -> torch.nn.Module:
  targets = lora_targets(model, module_path)
  if not targets:
    raise ValueError(f"module_path {module_path!r} matched no projection")
  for mod, slice_name, _ in targets:
    mod.add_lora(slice_name, rank, alpha, dtype=dtype)
  for p in model.parameters():
    if not getattr(p, "is_lora", False):
      p.requires_grad_(False)
  if weight_qtype:
    from . import qlora
    qlora.quantize_frozen_weights(model, weight_qtype, tile_size, only=[t[0] for t in targets])
  return model


def is_lora_enabled(model: torch.nn.Module) -> bool:
  return any(getattr(p, "is_lora", False) for p in model.parameters())


@torch.no_grad()
def merge_lora(model: torch.nn.Module) -> torch.nn.Module:
  """W += B A * alpha / rank for every adapter, then removes the adapters
  (tunix/models/safetensors_saver.py:90-112)."""
  for mod in model.modules():
    if not isinstance(mod, Linear) or not len(mod.lora_a):
      continue
    w = mod.weight().detach().float().clone()
    for key in list(mod.lora_a.keys()):
      lo, hi = mod.slices["" if key == "w" else key]
      w[lo:hi] += (mod.lora_b[key].float() @ mod.lora_a[key].float()) * mod.lora_scale[key]
    mod.quant = None
    mod.w.data = w.to(mod.w.dtype)
    mod.lora_a.clear()
    mod.lora_b.clear()
    mod.lora_scale.clear()
  return model
