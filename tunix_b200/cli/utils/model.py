"""Model and tokenizer construction from config sections (tunix/cli/utils/model.py:31-216)."""
from __future__ import annotations

import logging
import os
from typing import Any, Dict, Mapping, Optional, Tuple

import torch

from ...generate import tokenizer_adapter as tokenizer_lib
from ...models import automodel, lora as lora_lib, naming

_DEFAULT_TOKENIZER_PATH = "meta-llama/Llama-3.1-8B"
_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
           "float16": torch.float16, "fp16": torch.float16}


def apply_lora_to_model(base_model, mesh, lora_config: Mapping[str, Any], rng_seed: int = 0):
  """LoRA (or QLoRA when `weight_qtype` is given) on the projections matched by `module_path`."""
  kw = {"module_path": lora_config["module_path"], "rank": lora_config["rank"], "alpha": lora_config["alpha"]}
  if "tile_size" in lora_config:
    kw["tile_size"] = lora_config["tile_size"]
  if "weight_qtype" in lora_config:
    kw["weight_qtype"] = lora_config["weight_qtype"]
  logging.info("%s is applied: %r", "Qlora" if "weight_qtype" in kw else "Lora", dict(lora_config))
  torch.manual_seed(rng_seed)
  model = lora_lib.apply_lora_to_model(base_model, **kw)
  if mesh is not None and getattr(mesh, "size", 1) > 1:
    from ...dist import fsdp
    fsdp.shard_model(model, mesh)
  return model


def resolve_tokenizer_path(model_config: Mapping[str, Any], tokenizer_path: str) -> str:
  src = model_config.get("model_source")
  if not src:
    return tokenizer_path
  family = naming.ModelNaming(model_name=model_config["model_name"]).model_family
  default = not tokenizer_path or tokenizer_path == _DEFAULT_TOKENIZER_PATH
  if family in ("gemma", "gemma1p1", "gemma2") and src == "kaggle":
    if not model_config.get("model_path"):
      raise ValueError("model_path is required for kaggle source")
    resolved = automodel.download_model(model_config["model_path"], model_config.get("model_download_path"),
                                        automodel.ModelSource(src))
    if default:
      return os.path.join(resolved, "tokenizer.model")
  elif default and model_config.get("model_path") and os.path.isdir(str(model_config["model_path"])):
    # a local checkpoint directory usually carries its tokenizer
    for f in ("tokenizer.model", "tokenizer.json"):
      if os.path.exists(os.path.join(model_config["model_path"], f)):
        return model_config["model_path"] if f.endswith(".json") else os.path.join(model_config["model_path"], f)
  return tokenizer_path


def create_tokenizer(tokenizer_config: Mapping[str, Any], tokenizer_path: Optional[str],
                     model_config: Optional[Mapping[str, Any]] = None):
  path = tokenizer_path or tokenizer_config["tokenizer_path"]
  if model_config is not None:
    path = resolve_tokenizer_path(model_config, path)
  return tokenizer_lib.Tokenizer(tokenizer_config["tokenizer_type"], path, tokenizer_config["add_bos"],
                                 tokenizer_config["add_eos"], os.environ.get("HF_TOKEN"))


def create_model(model_config: Mapping[str, Any], tokenizer_config: Mapping[str, Any], mesh) -> Tuple[Any, str]:
  """-> (model, tokenizer path). Sources: local/hub safetensors, Orbax directory, random init."""
  tokenizer_path = resolve_tokenizer_path(model_config, tokenizer_config["tokenizer_path"])
  src = model_config["model_source"] or "dummy"
  try:
    source = automodel.ModelSource(src)
  except ValueError as e:
    raise ValueError(f"Unsupported model source: {src}. Available sources: "
                     f"{[s.value for s in automodel.ModelSource]}") from e
  dtype = _DTYPES.get(str(model_config.get("dtype") or model_config.get("load_dtype") or "bfloat16").lower())
  if dtype is None:
    raise ValueError(f"Invalid dtype: {model_config.get('dtype')}")
  kw: Dict[str, Any] = {}
  if model_config.get("model_overrides"):
    import dataclasses
    cfg = automodel.call_model_config(naming.ModelNaming(model_id=model_config["model_id"]).model_name)
    kw["model_config"] = dataclasses.replace(cfg, **model_config["model_overrides"])
  model, _ = automodel.AutoModel.from_pretrained(
      model_id=model_config["model_id"], mesh=mesh, model_source=source,
      model_download_path=model_config.get("model_download_path"), model_path=model_config.get("model_path") or None,
      rng_seed=model_config.get("rng_seed", 0), dtype=dtype, device=model_config.get("device"), **kw)
  if model_config.get("lora_config"):
    model = apply_lora_to_model(model, mesh, model_config["lora_config"], rng_seed=model_config.get("rng_seed", 0))
  else:
    logging.info("Training with Full Weight")
  if model_config.get("model_display"):
    print(model)
  return model, tokenizer_path
