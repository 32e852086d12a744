"""DeepScaleR math data for the agentic GRPO recipe (tunix/cli/recipes/deepscaler_data.py:27-76).

`create_dataset(train_data_path, eval_data_path)` reads the DeepScaleR training problems (a JSON array or JSON
lines with `problem` / `answer`) and returns a random-access dataset whose elements have the keys the RL pipeline
expects: `prompts` (question plus the boxed-answer instruction), `question`, `answer`. The evaluation file (AIME,
parquet or JSON) is validated and exposed through `create_eval_dataset`; both are read with pandas / pyarrow from
local paths (no remote file systems in this build).
"""
from __future__ import annotations

import json
import os
from typing import Any, Dict, List

from ...data.dataset import ListDataset

INSTRUCTION = "Let's think step by step, and put your final answer within \\boxed{}."


def _records(path: str) -> List[Dict[str, Any]]:
  if not os.path.isfile(path):
    raise FileNotFoundError(f"dataset file not found: {path}")
  if path.endswith(".parquet"):
    import pyarrow.parquet as pq
    return pq.read_table(path).to_pylist()
  with open(path, encoding="utf-8") as f:
    text = f.read()
  if path.endswith(".jsonl"):
    return [json.loads(line) for line in text.splitlines() if line.strip()]
  loaded = json.loads(text)
  return loaded if isinstance(loaded, list) else list(loaded.get("data", []))


def to_prompt(record: Dict[str, Any]) -> Dict[str, Any]:
  question = record.get("question", record.get("problem", ""))
  return {"prompts": f"{question} {INSTRUCTION}", "question": question,
          "answer": record.get("answer", record.get("ground_truth", ""))}


def create_dataset(train_data_path: str, eval_data_path: str = "", shuffle: bool = False, seed: int = 42) -> ListDataset:
  """The training set; `eval_data_path`, when given, must exist (it is read by `create_eval_dataset`)."""
  if eval_data_path and not os.path.isfile(eval_data_path):
    raise FileNotFoundError(f"evaluation file not found: {eval_data_path}")
  train = ListDataset(_records(train_data_path))
  if shuffle:
    train = train.shuffle(seed)
  return train.map(to_prompt)


def create_eval_dataset(eval_data_path: str) -> ListDataset:
  return ListDataset(_records(eval_data_path)).map(to_prompt)
