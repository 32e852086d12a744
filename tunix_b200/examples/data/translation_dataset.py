"""Translation SFT data (role of tunix/examples/data/translation_dataset.py:39-230).

Records are `{"src": ..., "dst": ...}` pairs read from a local `.jsonl` / `.json` / `.parquet`
file or directory (`<name>/train.*`, `<name>/validation.*`), or generated synthetically when
`dataset_name == "synthetic"`. Each pair becomes `"Translate this into French:\n<src>\n"` +
`<dst>`, tokenised with BOS/EOS, right-padded to `max_target_length`; the loss mask covers the
target tokens only; over-long examples are dropped.
"""
from __future__ import annotations

import json
import os
from typing import Any, Dict, Iterable, List, Optional, Tuple

import numpy as np

from ...data import ListDataset
from ...sft.peft_trainer import TrainingInput

INPUT_TEMPLATE = {"prefix": "Translate this into French:\n", "suffix": "\n"}


def _read_records(path: str) -> List[Dict[str, Any]]:
  if path.endswith(".jsonl"):
    with open(path) as f:
      return [json.loads(l) for l in f if l.strip()]
  if path.endswith(".json"):
    with open(path) as f:
      return json.load(f)
  if path.endswith(".parquet"):
    import pyarrow.parquet as pq
    return pq.read_table(path).to_pylist()
  raise ValueError(f"unsupported data file {path}")


def _load_split(name_or_path: str, split: str) -> List[Dict[str, Any]]:
  if os.path.isfile(name_or_path):
    return _read_records(name_or_path) if split == "train" else []
  for ext in (".jsonl", ".json", ".parquet"):
    p = os.path.join(name_or_path, split + ext)
    if os.path.exists(p):
      return _read_records(p)
  return []


def _synthetic(n: int, seed: int = 0) -> List[Dict[str, str]]:
  rng = np.random.default_rng(seed)
  words = ["alpha", "beta", "gamma", "delta", "epsilon", "zeta", "eta", "theta", "iota", "kappa"]
  out = []
  for _ in range(n):
    k = int(rng.integers(3, 9))
    src = [words[int(i)] for i in rng.integers(0, len(words), k)]
    out.append({"src": " ".join(src), "dst": " ".join(w[::-1] for w in src)})
  return out


def _pair(rec: Dict[str, Any]) -> Tuple[str, str]:
  if "translation" in rec:                       # opus-100 style {"translation": {"en": .., "fr": ..}}
    vals = list(rec["translation"].values())
    return vals[0], vals[1]
  return rec["src"], rec["dst"]


def build_example(rec: Dict[str, Any], tokenizer, max_len: int) -> Optional[Dict[str, np.ndarray]]:
  src, dst = _pair(rec)
  s = tokenizer.tokenize(src, prefix=INPUT_TEMPLATE["prefix"], suffix=INPUT_TEMPLATE["suffix"], add_eos=False)
  d = tokenizer.tokenize(dst, add_eos=True)
  if len(d) and tokenizer.bos_id() and d[0] == tokenizer.bos_id():
    d = d[1:]
  n = len(s) + len(d)
  if n > max_len:
    return None
  pad = tokenizer.pad_id() or 0
  toks = np.full(max_len, pad, dtype=np.int64)
  mask = np.zeros(max_len, dtype=np.int64)
  toks[:len(s)] = s
  toks[len(s):n] = d
  mask[len(s):n] = 1
  return {"input_tokens": toks, "input_mask": mask}


def _to_batches(records, tokenizer, batch_size: int, max_len: int, epochs: Optional[int]):
  examples = [e for e in (build_example(r, tokenizer, max_len) for r in records) if e is not None]
  ds = ListDataset(examples).repeat(epochs or 1)
  return ds.to_iter_dataset().batch(batch_size, drop_remainder=True).map(
      lambda b: TrainingInput(input_tokens=b["input_tokens"], input_mask=b["input_mask"]))


def create_datasets(dataset_name: str, global_batch_size: int, max_target_length: int, num_train_epochs: Optional[int],
                    tokenizer, tfds_download: bool = False, num_synthetic: int = 256):
  """-> (train batches, eval batches) of `TrainingInput`."""
  if dataset_name == "synthetic":
    train, evl = _synthetic(num_synthetic, 0), _synthetic(max(global_batch_size, 16), 1)
  else:
    train = _load_split(dataset_name, "train")
    evl = _load_split(dataset_name, "validation") or _load_split(dataset_name, "test")
    if not train:
      raise FileNotFoundError(f"no train split found at {dataset_name!r}: expected a .jsonl/.json/.parquet file or a "
                              "directory with train.* (there is no dataset download on this platform)")
  return (_to_batches(train, tokenizer, global_batch_size, max_target_length, num_train_epochs),
          _to_batches(evl, tokenizer, global_batch_size, max_target_length, 1) if evl else None)
