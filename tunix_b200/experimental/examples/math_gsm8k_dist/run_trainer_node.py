"""Trainer node of the distributed GSM8K GRPO example
(tunix/experimental/examples/math_gsm8k_dist/run_trainer_node.py).

Hosts the policy being trained behind a `TrainerWorker` (step-level `PeftTrainerV2`), serves it over remote
execution, and is the SOURCE of weight transfers: its parameters are exposed through a host-staged endpoint that
rollout nodes pull from when the coordinator says so. The loss is not chosen here: the control plane sends it
(`with_loss_fn`) once it knows the algorithm's configuration.

  python -m tunix_b200.experimental.examples.math_gsm8k_dist.run_trainer_node \\
      --model tiny --port 50071 --discovery_addrs=control:50070 --lr 1e-2
"""
from __future__ import annotations

import argparse
import sys

from . import models, node_common


def build_worker(args: argparse.Namespace):
  from tunix_b200 import optim
  from tunix_b200.common.configs import TrainingConfig
  from ...orchestrator import host_staged_handler
  from ...train import peft_trainer_v2
  from ...worker import trainer_worker
  model = models.build_model(args.model, args.seed, args.weights)
  if args.lora_rank:
    from tunix_b200.models import lora
    lora.apply_lora_to_model(model, rank=args.lora_rank, alpha=float(2 * args.lora_rank))
  endpoint = host_staged_handler.HostStagedEndpoint()

  def make_trainer():
    config = TrainingConfig(eval_every_n_steps=10**9, pbar_description=None, max_steps=None,
                            checkpoint_root_directory=args.checkpoint_dir)
    return peft_trainer_v2.PeftTrainerV2(model, optim.adamw(args.lr), config)
  worker = trainer_worker.TrainerWorker(make_trainer, worker_id=args.worker_id or "trainer-0", handler=endpoint)
  return worker, endpoint


def main(ctx, argv) -> None:
  parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
  node_common.common_flags(parser, default_port=50071)
  parser.add_argument("--lr", type=float, default=1e-5)
  parser.add_argument("--lora_rank", type=int, default=0)
  parser.add_argument("--checkpoint_dir", default=None)
  args = parser.parse_args(argv)
  worker, endpoint = build_worker(args)
  node_common.serve_and_wait(ctx, worker, args, "actor", endpoint, worker.work_unit)


if __name__ == "__main__":
  node_common.run_standalone(f"{__spec__.name}.main" if __spec__ else "run_trainer_node.main", sys.argv[1:])
