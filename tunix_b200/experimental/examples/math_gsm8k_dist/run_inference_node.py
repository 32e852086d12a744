"""Inference node of the distributed GSM8K GRPO example
(tunix/experimental/examples/math_gsm8k_dist/run_inference_node.py).

Hosts the frozen reference policy behind an `InferenceWorker` and answers per-token log-prob requests, which the
control plane needs only when the KL coefficient is non-zero. It takes no part in weight transfers: the reference
never changes.

  python -m tunix_b200.experimental.examples.math_gsm8k_dist.run_inference_node \\
      --model tiny --port 50073 --discovery_addrs=control:50070 --micro_batch_size 8
"""
from __future__ import annotations

import argparse
import sys

from . import models, node_common


def build_worker(args: argparse.Namespace):
  from ...worker import inference_worker
  model = models.build_model(args.model, args.seed, args.weights)
  for p in model.parameters():
    p.requires_grad_(False)
  pad, eos = models.pad_and_eos(models.build_tokenizer(args.model, args.tokenizer))
  return inference_worker.InferenceWorker({"reference": model}, pad_id=pad, eos_id=eos,
                                          worker_id=args.worker_id or "inference-0",
                                          micro_batch_size=args.micro_batch_size or None)


def main(ctx, argv) -> None:
  parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
  node_common.common_flags(parser, default_port=50073)
  parser.add_argument("--micro_batch_size", type=int, default=0)
  args = parser.parse_args(argv)
  node_common.serve_and_wait(ctx, build_worker(args), args, "reference")


if __name__ == "__main__":
  node_common.run_standalone(f"{__spec__.name}.main" if __spec__ else "run_inference_node.main", sys.argv[1:])
