"""Helpers shared by the family packages: preset registration and model subclasses."""
from __future__ import annotations

from typing import Callable, Dict

import torch

from .transformer import ModelConfig, Transformer


class PresetMeta(type):
  """Lets `ModelConfig.qwen3_8b()` style classmethod presets live in a plain dict."""

  def __getattr__(cls, name: str):
    presets: Dict[str, Callable[[], ModelConfig]] = cls.__dict__.get("_presets", {})
    if name in presets:
      return presets[name]
    raise AttributeError(f"{cls.__name__} has no preset {name!r}; available: {sorted(presets)}")

  def __dir__(cls):
    return list(super().__dir__()) + list(cls.__dict__.get("_presets", {}))


def make_family(family: str, defaults: dict, presets: Dict[str, dict], aliases: Dict[str, str] = None):
  """Builds the `ModelConfig` namespace of a family: calling it constructs a config with the
  family defaults, and every preset name is a zero-argument factory."""
  aliases = aliases or {}

  def build(**kw) -> ModelConfig:
    merged = dict(defaults)
    merged.update(kw)
    # the reference spells these differently in some families
    if "num_embed" in merged:
      merged["vocab_size"] = merged.pop("num_embed")
    if "use_tied_embedding" in merged:
      merged["weight_tying"] = merged.pop("use_tied_embedding")
    return ModelConfig(family=family, **merged)

  table = {name: (lambda kw=kw: build(**kw)) for name, kw in presets.items()}
  for alias, target in aliases.items():
    table[alias] = table[target]

  class FamilyConfig(metaclass=PresetMeta):
    _presets = table

    def __new__(cls, **kw):
      return build(**kw)

    @classmethod
    def preset_names(cls):
      return sorted(table)

  FamilyConfig.__name__ = "ModelConfig"
  FamilyConfig.__qualname__ = f"{family}.ModelConfig"
  return FamilyConfig
