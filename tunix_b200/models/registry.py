"""Catalogue of supported checkpoints (role of tunix/models/registry.py:19-536).

Each entry ties a Hugging Face id to the preset that builds its config. The table is generated
from the presets the family packages register, so a preset added there shows up here.
"""
from __future__ import annotations

import importlib
from typing import Callable, Dict, List, Optional, Tuple

from . import naming

_CATEGORIES = ("gemma", "gemma3", "gemma4", "llama3", "qwen2", "qwen3")

# organisation and exact spelling on the hub, by family
_HF_FORMAT: Dict[str, Callable[[str], str]] = {
    "gemma": lambda v: f"google/gemma-{v}", "gemma1p1": lambda v: f"google/gemma-1.1-{v}",
    "gemma2": lambda v: f"google/gemma-2-{v}", "gemma3": lambda v: f"google/gemma-3-{v}",
    "gemma4": lambda v: f"google/gemma-4-{v}",
    "llama3": lambda v: f"meta-llama/Meta-Llama-3-{v}", "llama3p1": lambda v: f"meta-llama/Llama-3.1-{v}",
    "llama3p2": lambda v: f"meta-llama/Llama-3.2-{v}",
    "qwen2p5": lambda v: f"Qwen/Qwen2.5-{v}", "qwen3": lambda v: f"Qwen/Qwen3-{v}",
    "qwen3p5": lambda v: f"Qwen/Qwen3.5-{v}",
    "deepseek_r1_distill_qwen": lambda v: f"deepseek-ai/DeepSeek-R1-Distill-Qwen-{v}",
}


def _version_to_hf(version: str) -> str:
  parts = version.split("_")
  out = []
  for p in parts:
    if p and p[0].isdigit():
      p = p.replace("p", ".")
      out.append(p.upper() if p[-1] in "bm" else p)
    else:
      out.append({"it": "it", "pt": "pt", "instruct": "Instruct", "base": "Base", "coder": "Coder",
                  "thinking": "Thinking"}.get(p, p))
  return "-".join(out)


def _config_module(category: str):
  return importlib.import_module(f"{__package__}.{category}.model")


def _build() -> Tuple[naming.ModelNaming, ...]:
  entries: List[naming.ModelNaming] = []
  for cat in _CATEGORIES:
    try:
      presets = _config_module(cat).ModelConfig.preset_names()
    except (ImportError, AttributeError):
      continue
    for config_id in presets:
      try:
        fam, ver = naming.get_model_family_and_version(config_id)
      except ValueError:
        continue
      fmt = _HF_FORMAT.get(fam)
      if fmt is None:
        continue
      hf_id = fmt(_version_to_hf(ver))
      try:
        n = naming.ModelNaming(model_id=hf_id)
      except ValueError:
        continue
      if n.model_config_id == config_id:
        entries.append(n)
  return tuple(entries)


MODEL_CATALOG: Tuple[naming.ModelNaming, ...] = _build()
_BY_CONFIG_ID = {m.model_config_id: m for m in MODEL_CATALOG}
_BY_HF_ID = {m.model_id.lower(): m for m in MODEL_CATALOG}


def lookup(model_id_or_config_id: str) -> Optional[naming.ModelNaming]:
  return _BY_HF_ID.get(model_id_or_config_id.lower()) or _BY_CONFIG_ID.get(model_id_or_config_id.lower())


def config_ids() -> List[str]:
  return sorted(_BY_CONFIG_ID)
