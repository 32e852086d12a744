"""Math word-problem prompts for RL (role of tunix/examples/data/math_dataset.py:44-200):
GSM8K-style records `{"question", "answer"}` where the gold answer follows `####`, rendered
either as chat messages under `prompt` (templating happens later) or as a finished string
under `prompts`."""
from __future__ import annotations

import json
import os
from typing import Any, Dict, List, Optional

import numpy as np

from ...data import ListDataset

SYSTEM_PROMPT = ("You are given a problem. Think about the problem and provide your reasoning. Place it between "
                 "<reasoning> and </reasoning>. Then, provide the final answer (i.e., just one numerical value) between "
                 "<answer> and </answer>.")
TEMPLATE = "<start_of_turn>user\n{system_prompt}\n\n{question}<end_of_turn>\n<start_of_turn>model\n"


def extract_hash_answer(text: str) -> Optional[str]:
  return text.split("####")[1].strip() if "####" in text else None


def apply_template(rec: Dict[str, Any], as_messages: bool = True, system_prompt: str = SYSTEM_PROMPT) -> Dict[str, Any]:
  q = rec["question"]
  ans = extract_hash_answer(rec["answer"]) if "####" in str(rec.get("answer", "")) else str(rec.get("answer", ""))
  base = {"question": q, "answer": ans}
  if as_messages:
    return {"prompt": [{"role": "system", "content": system_prompt}, {"role": "user", "content": q}], **base}
  return {"prompts": TEMPLATE.format(system_prompt=system_prompt, question=q), **base}


def _synthetic(n: int, seed: int) -> List[Dict[str, str]]:
  rng = np.random.default_rng(seed)
  out = []
  for _ in range(n):
    a, b = int(rng.integers(1, 50)), int(rng.integers(1, 50))
    out.append({"question": f"What is {a} + {b}?", "answer": f"{a} plus {b} #### {a + b}"})
  return out


def create_dataset(name: str = "synthetic", split: str = "train", data_dir: str = "", as_messages: bool = True,
                   num_synthetic: int = 128, seed: int = 0, **unused) -> ListDataset:
  if name == "synthetic":
    recs = _synthetic(num_synthetic, seed + (split != "train"))
  else:
    path = name if os.path.exists(name) else os.path.join(data_dir, name)
    if os.path.isdir(path):
      path = next((os.path.join(path, split + e) for e in (".jsonl", ".json", ".parquet")
                   if os.path.exists(os.path.join(path, split + e))), path)
    if not os.path.isfile(path):
      raise FileNotFoundError(f"dataset {name!r} not found locally (looked at {path})")
    if path.endswith(".parquet"):
      import pyarrow.parquet as pq
      recs = pq.read_table(path).to_pylist()
    else:
      with open(path) as f:
        recs = [json.loads(l) for l in f if l.strip()] if path.endswith(".jsonl") else json.load(f)
  return ListDataset(recs).map(lambda r: apply_template(r, as_messages))
