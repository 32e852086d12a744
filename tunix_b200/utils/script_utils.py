"""Helpers for example scripts: question/answer datasets from local files, train/eval split,
and a profiling context (tunix/utils/script_utils.py:35-175).

Datasets are read from disk (a `.json` list, a `.jsonl` file, or a directory that holds
`<split>.json[l]`); nothing is downloaded.
"""
from __future__ import annotations

import contextlib
import json
import logging
import os
from typing import Any, Callable, Dict, List, Optional, Tuple

from ..data import dataset as dataset_lib

log = logging.getLogger(__name__)


def _read_records(path: str, split: str) -> List[Dict[str, Any]]:
  if os.path.isdir(path):
    for ext in (".jsonl", ".json"):
      cand = os.path.join(path, split + ext)
      if os.path.isfile(cand):
        path = cand
        break
    else:
      raise FileNotFoundError(f"no {split}.json or {split}.jsonl under {path}")
  with open(path, "r", encoding="utf-8") as f:
    if path.endswith(".jsonl"):
      return [json.loads(line) for line in f if line.strip()]
    data = json.load(f)
  if isinstance(data, dict):
    data = data.get(split, data.get("data", []))
  return list(data)


def _as_text(v) -> str:
  return v if isinstance(v, str) else v.decode("utf-8")


def get_dataset(path: str, split: str, seed: int, system_prompt: str, *,
                answer_extractor: Callable[[str], Optional[str]], dataset_name: str = "gsm8k"):
  """Shuffled dataset of {"prompts", "question", "answer"}; records need "question" and "answer"."""
  del dataset_name
  records = _read_records(path, split)
  return dataset_lib.ListDataset(records).shuffle(seed=seed).map(lambda x: {
      "prompts": system_prompt + _as_text(x["question"]),
      "question": system_prompt + _as_text(x["question"]),
      "answer": answer_extractor(_as_text(x["answer"])),
  })


def get_train_and_eval_datasets(data_path: str, split: str, seed: int, system_prompt: str, batch_size: int,
                                num_batches: Optional[int], train_fraction: float, num_epochs: Optional[int], *,
                                answer_extractor: Callable[[str], Optional[str]], dataset_name: str = "gsm8k"):
  ds = get_dataset(data_path, split, seed, system_prompt, answer_extractor=answer_extractor,
                   dataset_name=dataset_name)
  n_batches = len(ds) // batch_size
  if num_batches:
    n_batches = min(n_batches, num_batches)
  ds = ds[:n_batches * batch_size]
  if train_fraction == 1.0:
    train, val = ds, None
  else:
    cut = int(n_batches * train_fraction) * batch_size
    train, val = ds[:cut], ds[cut:]
  if num_epochs:
    train = train.repeat(num_epochs)
    val = val.repeat(num_epochs) if val is not None else None
  return train.batch(batch_size), (val.batch(batch_size) if val is not None else None)


class profile_and_capture_log:   # pylint: disable=invalid-name
  """`with profile_and_capture_log("tag", log_dir=...)`: a torch profiler trace of the block
  (CPU + CUDA activities, Chrome trace under `log_dir`) when `enable_profile`, else a no-op."""

  def __init__(self, tag: str = "", enable_profile: bool = True, log_dir: Optional[str] = None, **_unused):
    self._tag = tag
    self._enable = enable_profile and log_dir is not None
    self._log_dir = log_dir
    self._prof = None

  def __enter__(self):
    if self._enable:
      import torch
      acts = [torch.profiler.ProfilerActivity.CPU]
      if torch.cuda.is_available():
        acts.append(torch.profiler.ProfilerActivity.CUDA)
      self._prof = torch.profiler.profile(activities=acts)
      self._prof.__enter__()
    return self

  def __exit__(self, exc_type, exc_value, traceback):
    if self._prof is not None:
      self._prof.__exit__(exc_type, exc_value, traceback)
      with contextlib.suppress(Exception):
        os.makedirs(self._log_dir, exist_ok=True)
        self._prof.export_chrome_trace(os.path.join(self._log_dir, f"{self._tag or 'profile'}.json"))
    return False
