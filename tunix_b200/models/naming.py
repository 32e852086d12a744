"""Model naming: Hugging Face id <-> config id <-> family / version / config category.

Same rules as tunix/models/naming.py:39-294: the model name is the last path element of the id,
lower-cased (`meta-llama-` prefix folded to `llama-`); the family is the longest known prefix;
the version is what follows, with '-' -> '_' and '.' -> 'p'; config id = `<family>_<version>`.
"""
from __future__ import annotations

import dataclasses
from typing import Dict, Optional, Tuple

_HF: Dict[str, Tuple[str, str]] = {          # prefix -> (family, config category)
    "gemma-": ("gemma", "gemma"), "gemma-1.1-": ("gemma1p1", "gemma"), "gemma-2-": ("gemma2", "gemma"),
    "gemma-3-": ("gemma3", "gemma3"), "gemma-4-": ("gemma4", "gemma4"),
    "llama-3-": ("llama3", "llama3"), "llama-3.1-": ("llama3p1", "llama3"), "llama-3.2-": ("llama3p2", "llama3"),
    "qwen2.5-": ("qwen2p5", "qwen2"), "qwen3-": ("qwen3", "qwen3"), "qwen3.5-": ("qwen3p5", "qwen3"),
    "deepseek-r1-distill-qwen-": ("deepseek_r1_distill_qwen", "qwen2"),
}
_CONFIG: Dict[str, Tuple[str, str]] = {
    (fam + "_"): (fam, cat) for fam, cat in _HF.values()
}


def _is_hf_name(name: str) -> bool:
  return "-" in name or "." in name or "/" in name


def _mapping(name: str) -> Dict[str, Tuple[str, str]]:
  if not name or any(c.isspace() for c in name):
    raise ValueError(f"Invalid model ID format: {name!r}. Expected a Huggingface model ID or a ConfigId.")
  return _HF if _is_hf_name(name) else _CONFIG


def split(model_name: str) -> Tuple[str, str]:
  """-> (raw family prefix, raw version) by longest matching family prefix."""
  model_name = model_name.lower()
  mapping = _mapping(model_name)
  best = max((f for f in mapping if model_name.startswith(f)), key=len, default="")
  if not best:
    raise ValueError(f"Could not determine model family for: {model_name}. Not one of the known families: "
                     f"{list(mapping)}")
  return best, model_name[len(best):].lstrip("-").lstrip("_") if mapping is _CONFIG else model_name[len(best):].lstrip("-")


def _std_version(raw: str) -> str:
  if not raw:
    return ""
  v = raw.lower().replace("-", "_").replace(".", "p")
  if len(v) > 1 and not v[0].isalnum():
    raise ValueError(f"Invalid model version format. Expected alphanumeric starting character, found: {v}")
  return v


def get_model_family_and_version(model_name: str) -> Tuple[str, str]:
  fam, ver = split(model_name)
  return _mapping(model_name.lower())[fam][0], _std_version(ver)


def get_model_config_category(model_name: str) -> str:
  fam, _ = split(model_name)
  return _mapping(model_name.lower())[fam][1]


def get_model_config_id(model_name: str) -> str:
  fam, ver = get_model_family_and_version(model_name)
  return f"{fam}_{ver}".replace(".", "p").replace("-", "_")


def get_model_name_from_model_id(model_id: str) -> str:
  if _is_hf_name(model_id):
    name = model_id.split("/")[-1].lower()
    if not name:
      raise ValueError(f"Invalid model ID format: {model_id!r}. Model name cannot be empty.")
    if name.startswith("meta-llama-"):
      name = name.replace("meta-llama-", "llama-", 1)
    return name
  return model_id.lower()


@dataclasses.dataclass(frozen=True)
class ModelNaming:
  model_id: Optional[str] = None
  model_name: Optional[str] = None
  model_family: Optional[str] = None
  model_version: Optional[str] = None
  model_config_category: Optional[str] = None
  model_config_id: Optional[str] = None

  def __post_init__(self):
    if self.model_id:
      name = get_model_name_from_model_id(self.model_id)
      if self.model_name and self.model_name != name:
        raise ValueError(f"model_name set in ModelNaming and one inferred from model_id do not match. model_name: "
                         f"{self.model_name} and model_id: {self.model_id}, model_name inferred from model_id: {name}.")
    else:
      name = self.model_name
    if not name:
      raise ValueError("Either model_name or model_id must be provided.")
    fam, ver = get_model_family_and_version(name)
    derived = {"model_name": name, "model_family": fam, "model_version": ver,
               "model_config_category": get_model_config_category(name), "model_config_id": get_model_config_id(name)}
    for field, value in derived.items():
      given = getattr(self, field)
      if field != "model_name" and given is not None and given != value:
        raise ValueError(f"{field} mismatch: {given} != {value}")
      object.__setattr__(self, field, value)
