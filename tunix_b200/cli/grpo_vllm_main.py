"""GRPO entry point with vLLM as the rollout engine (tunix/cli/grpo_vllm_main.py:14-24).

The reference's variant exists to start the trainer under vLLM's application runner. Here vLLM runs in-process
(`generate/vllm_sampler.py`), so the entry point is `grpo_main` with `rollout_engine=vllm` forced unless the command
line already picks an engine, after checking that vLLM imports - failing at start, not at the first rollout.

  python -m tunix_b200.cli.grpo_vllm_main base_config.yaml model_config.model_source=... rollout_config.rollout_vllm_hbm_utilization=0.4
"""
from __future__ import annotations

import logging
import sys
from typing import List

from . import grpo_main


def with_vllm_engine(argv: List[str]) -> List[str]:
  if any(a.startswith("rollout_engine=") for a in argv[1:]):
    return list(argv)
  return list(argv) + ["rollout_engine=vllm"]


def main(argv, **kwargs):
  try:
    import vllm  # noqa: F401
  except Exception as e:  # noqa: BLE001
    raise SystemExit(f"grpo_vllm_main needs an importable vllm package: {type(e).__name__}: {e}")
  return grpo_main.main(with_vllm_engine(argv), **kwargs)


if __name__ == "__main__":
  logging.basicConfig(level=logging.INFO)
  main(sys.argv)
