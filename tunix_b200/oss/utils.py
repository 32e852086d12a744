"""Download helpers (tunix/oss/utils.py:24-95): fetch a checkpoint directory from the Hugging Face hub, Kaggle or a
`gs://` bucket into a local folder and return its path. Every backend package is optional and imported on use; a
missing package or an unreachable network raises `FileNotFoundError` that names the local-path alternative, so
offline runs fail with one clear message instead of a hang."""
from __future__ import annotations

import os
import shutil
from typing import Optional


def pathways_available() -> bool:
  """The reference probes for a Pathways proxy; this framework runs one process per GPU and never has one."""
  return False


def _unreachable(what: str, e: BaseException) -> FileNotFoundError:
  return FileNotFoundError(f"{what} could not be fetched ({type(e).__name__}: {e}); download it on a connected "
                           "machine and pass the local directory instead")


def load_file_from_gcs(file_dir: str, target_dir: Optional[str] = None) -> str:
  """Copies `gs://bucket/dir` (recursively) under `target_dir` (default: a cache folder in $TMPDIR) and returns the
  local path; anything that is not a `gs://` URL is returned unchanged."""
  if not file_dir.startswith("gs://"):
    return file_dir
  import tempfile
  target_dir = target_dir or os.path.join(tempfile.gettempdir(), "tunix_b200_gcs")
  local = os.path.join(target_dir, file_dir[len("gs://"):].strip("/").replace("/", "_"))
  if os.path.isdir(local) and os.listdir(local):
    return local
  os.makedirs(local, exist_ok=True)
  try:
    import fsspec
    fs = fsspec.filesystem("gs")
    fs.get(file_dir.rstrip("/") + "/", local + "/", recursive=True)
  except Exception as e:  # pylint: disable=broad-exception-caught
    shutil.rmtree(local, ignore_errors=True)
    raise _unreachable(file_dir, e) from e
  return local


def kaggle_pipeline(model_id: str, model_download_path: Optional[str] = None) -> str:
  """Downloads a Kaggle model handle (e.g. `google/gemma-2/flax/gemma2-2b-it`) and returns its directory."""
  try:
    import kagglehub
    if model_download_path:
      os.environ.setdefault("KAGGLEHUB_CACHE", model_download_path)
    return kagglehub.model_download(model_id)
  except Exception as e:  # pylint: disable=broad-exception-caught
    raise _unreachable(f"Kaggle model {model_id!r}", e) from e


def hf_pipeline(model_id: str, model_download_path: Optional[str] = None) -> str:
  """Downloads the weight, config and tokenizer files of a hub repository and returns the directory."""
  try:
    import huggingface_hub as hf
    return hf.snapshot_download(repo_id=model_id, local_dir=model_download_path,
                                allow_patterns=["*.safetensors", "*.json", "tokenizer*", "*.model"])
  except Exception as e:  # pylint: disable=broad-exception-caught
    raise _unreachable(f"Hugging Face repository {model_id!r}", e) from e
