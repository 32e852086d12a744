"""Agentic GRPO on DeepScaleR-style math data through the command-line pipeline.

  python examples/deepscaler/train_deepscaler.py --train deepscaler.json --eval aime.parquet \\
      --tokenizer /path/to/tokenizer.model [key=value overrides of cli/base_agentic_config.yaml ...]

The data recipe is `tunix_b200.cli.recipes.deepscaler_data` (prompt = problem + boxed-answer instruction); the model,
mesh, rollout engine and optimizer come from the YAML config and the overrides, exactly as with
`python -m tunix_b200.cli.grpo_main`. Without `--train` a few synthetic problems are written to a temporary file,
which is enough to see the whole loop run on CPU with `model_config.model_source=dummy`.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import tempfile

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from tunix_b200.cli import grpo_main


def synthetic_problems(path: str, n: int = 16) -> None:
  rows = [{"problem": f"What is {a} plus {b}?", "answer": str(a + b)} for a, b in ((i, 2 * i + 1) for i in range(n))]
  with open(path, "w", encoding="utf-8") as f:
    json.dump(rows, f)


def main() -> None:
  ap = argparse.ArgumentParser()
  ap.add_argument("--train", default="")
  ap.add_argument("--eval", default="")
  ap.add_argument("--tokenizer", required=True)
  ap.add_argument("--tokenizer-type", default="sentencepiece")
  args, overrides = ap.parse_known_args()
  tmp = None
  if not args.train:
    tmp = tempfile.TemporaryDirectory()
    args.train = os.path.join(tmp.name, "deepscaler.json")
    synthetic_problems(args.train)
  call = f"tunix_b200.cli.recipes.deepscaler_data:create_dataset(train_data_path={args.train!r}, eval_data_path={args.eval!r})"
  argv = ["grpo_main", "base_agentic_config.yaml", "training_mode=agentic_grpo", f"data_module={call}",
          f"tokenizer_config.tokenizer_path={args.tokenizer}", f"tokenizer_config.tokenizer_type={args.tokenizer_type}",
          *overrides]
  grpo_main.main(argv)
  if tmp is not None:
    tmp.cleanup()


if __name__ == "__main__":
  main()
