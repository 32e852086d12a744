"""`AutoModel.from_pretrained`: model id -> config preset -> weights (tunix/models/automodel.py:384-627).

Sources: a local directory of Hugging Face safetensors (`HUGGINGFACE` with `model_path`, or a
hub id that is already present in the local cache / download path), a checkpoint in the
reference's Orbax layout (`ORBAX`), or random weights (`DUMMY`). Hub, Kaggle and GCS downloads
need network access and are delegated to `huggingface_hub` / `kagglehub` when those are
importable and reachable; otherwise the error names the directory that was searched.
"""
from __future__ import annotations

import enum
import importlib
import os
from typing import Any, Optional, Tuple

import torch

from . import dummy_model_creator, naming, safetensors_loader
from .transformer import Transformer


class ModelModule(enum.Enum):
  MODEL = "model"
  PARAMS = "params"
  PARAMS_SAFETENSORS = "params_safetensors"


class ModelSource(enum.Enum):
  KAGGLE = "kaggle"
  GCS = "gcs"
  HUGGINGFACE = "huggingface"
  INTERNAL = "internal"
  MAXTEXT = "maxtext"
  ORBAX = "orbax"
  DUMMY = "dummy"


def get_model_module(model_name: str, module_type: ModelModule = ModelModule.MODEL) -> Any:
  n = naming.ModelNaming(model_name=model_name) if "/" not in model_name else naming.ModelNaming(model_id=model_name)
  mod = "model" if module_type != ModelModule.MODEL else module_type.value
  try:
    return importlib.import_module(f"{__package__}.{n.model_config_category}.{mod}")
  except ImportError as e:
    raise ValueError(f"Unsupported model family {n.model_config_category!r} for {model_name!r}") from e


def call_model_config(model_name: str) -> Any:
  """Config object of a model name / HF id / config id, e.g. `call_model_config("qwen3-8b")`."""
  n = naming.ModelNaming(model_name=model_name) if "/" not in model_name else naming.ModelNaming(model_id=model_name)
  cfg_cls = get_model_module(n.model_name).ModelConfig
  try:
    return getattr(cfg_cls, n.model_config_id)()
  except AttributeError as e:
    raise ValueError(f"No config preset {n.model_config_id!r} in family {n.model_config_category!r}; available: "
                     f"{cfg_cls.preset_names()}") from e


def download_model(model_id_or_path: str, model_download_path: Optional[str], model_source: ModelSource) -> str:
  """Returns a local directory with the checkpoint files."""
  if os.path.exists(model_id_or_path):
    return model_id_or_path
  if model_download_path:
    cand = os.path.join(model_download_path, model_id_or_path.split("/")[-1])
    if os.path.isdir(cand):
      return cand
  if model_source == ModelSource.HUGGINGFACE:
    try:
      from huggingface_hub import snapshot_download
      return snapshot_download(repo_id=model_id_or_path, local_dir=model_download_path,
                               allow_patterns=["*.safetensors", "*.json", "tokenizer*"])
    except Exception as e:  # no network, no package, or not cached
      raise FileNotFoundError(f"{model_id_or_path!r} is not a local path and could not be fetched from the hub "
                              f"({type(e).__name__}: {e}); pass model_path=<directory with *.safetensors>") from e
  if model_source == ModelSource.KAGGLE:
    try:
      import kagglehub
      return kagglehub.model_download(model_id_or_path)
    except Exception as e:
      raise FileNotFoundError(f"Kaggle download of {model_id_or_path!r} failed: {e}") from e
  raise FileNotFoundError(f"model path {model_id_or_path!r} does not exist (source {model_source.value})")


def create_model_from_safe_tensors(model_name: str, file_dir: str, model_config: Any = None, mesh=None,
                                   dtype: Optional[torch.dtype] = None, device: Optional[str] = None) -> Transformer:
  cfg = model_config or call_model_config(model_name)
  device = device or ("cuda" if torch.cuda.is_available() else "cpu")
  return safetensors_loader.load_and_create_model(file_dir, Transformer, cfg, mesh, dtype=dtype, device=device)


class AutoModel:
  @classmethod
  def from_pretrained(cls, model_id: str, mesh=None, *, model_source: ModelSource = ModelSource.HUGGINGFACE,
                      model_path: Optional[str] = None, model_download_path: Optional[str] = None,
                      dtype: Optional[torch.dtype] = torch.bfloat16, device: Optional[str] = None,
                      **kwargs) -> Tuple[Transformer, Optional[str]]:
    """-> (model, resolved local path). `mesh` (a `dist.mesh.Mesh`) shards the result when given."""
    n = naming.ModelNaming(model_id=model_id)
    cfg = kwargs.pop("model_config", None) or call_model_config(n.model_name)
    device = device or ("cuda" if torch.cuda.is_available() else "cpu")
    model_cls = Transformer
    if n.model_config_category == "gemma4":
      from .gemma4 import Gemma4
      model_cls = Gemma4
      if model_source not in (ModelSource.DUMMY,):
        raise NotImplementedError("Gemma 4 weights: only random initialisation (model_source=DUMMY) is wired up; "
                                  "the safetensors key map of this family is not written yet")
      cfg = cfg.replace(dtype=dtype) if dtype is not None else cfg
    if model_source == ModelSource.DUMMY:
      model = dummy_model_creator.create_dummy_model(model_cls, cfg, mesh, dtype=dtype, device=device,
                                                     random_seed=kwargs.pop("rng_seed", 0))
      resolved = None
    else:
      if not model_path and model_source in (ModelSource.INTERNAL, ModelSource.GCS, ModelSource.KAGGLE,
                                             ModelSource.ORBAX):
        raise ValueError(f"model_path is required for model_source: {model_source}. Please provide a valid "
                         "model_path.")
      if model_source == ModelSource.MAXTEXT:
        raise NotImplementedError("MaxText checkpoints are converted offline to the Orbax layout; load them with "
                                  "model_source=ModelSource.ORBAX")
      resolved = download_model(model_path or model_id, model_download_path, model_source)
      if model_source == ModelSource.ORBAX:
        from ..ckpt import layout, orbax_layout
        model = dummy_model_creator.create_dummy_model(Transformer, cfg, mesh, dtype=dtype, device=device)
        tree = orbax_layout.read_tree(resolved)
        layout.tree_to_model(model, tree)
      else:
        model = create_model_from_safe_tensors(n.model_name, resolved, cfg, mesh, dtype=dtype, device=device)
    if mesh is not None and getattr(mesh, "size", 1) > 1:
      from ..dist import fsdp
      fsdp.shard_model(model, mesh)
    return model, resolved
