"""Direct preference optimisation on synthetic preference pairs, with the reference policy sharing the backbone.

  python examples/dpo/dpo_synthetic.py --steps 20
  python examples/dpo/dpo_synthetic.py --algorithm orpo --steps 20       # no reference model at all

Pairs prefer polite answers over rude ones. With `--lora-rank` the policy is the backbone plus adapters and the
reference is the same backbone with the adapters switched off, so no second copy of the weights exists. Printed: the
loss, the reward margin (chosen minus rejected, in units of beta * log-ratio) and the preference accuracy.
"""
from __future__ import annotations

import argparse
import copy
import os
import random
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import _common
from tunix_b200 import optim
from tunix_b200.models import lora as lora_lib
from tunix_b200.sft.dpo import dpo_trainer as dpo

QUESTIONS = ["how do I reset my password", "where is my order", "can you explain the invoice", "is the store open"]
POLITE = ["happy to help, here is how", "of course, let me check that for you", "certainly, one moment please"]
RUDE = ["figure it out yourself", "not my problem", "read the manual"]


def pairs(n: int, batch: int, seed: int = 0):
  rng = random.Random(seed)
  for _ in range(n):
    qs = [rng.choice(QUESTIONS) for _ in range(batch)]
    yield dpo.DataInput(prompts=qs, chosen_responses=[rng.choice(POLITE) for _ in qs],
                        rejected_responses=[rng.choice(RUDE) for _ in qs])


def main() -> None:
  ap = argparse.ArgumentParser()
  ap.add_argument("--algorithm", choices=("dpo", "orpo"), default="dpo")
  ap.add_argument("--steps", type=int, default=20)
  ap.add_argument("--beta", type=float, default=0.1)
  ap.add_argument("--lora-rank", type=int, default=0)
  args = ap.parse_args()
  dev = _common.device()
  policy = _common.tiny(layers=2, width=64).to(dev)
  if args.algorithm == "orpo":
    reference = None
  elif args.lora_rank:
    lora_lib.apply_lora_to_model(policy, rank=args.lora_rank, alpha=2.0 * args.lora_rank)
    reference = dpo.ReferenceWithAdaptersOff(policy)     # a view of the same backbone; holds no parameters
  else:
    reference = copy.deepcopy(policy)
  config = dpo.DPOTrainingConfig(algorithm=args.algorithm, beta=args.beta, max_steps=args.steps, eval_every_n_steps=10**9,
                                 pbar_description=None, max_prompt_length=40, max_response_length=48)
  trainer = dpo.DPOTrainer(policy, reference, optim.adamw(3e-3), config, tokenizer=_common.CharTokenizer())
  trainer.train(list(pairs(args.steps, 4)))
  for name in ("loss", "rewards/margin", "rewards/accuracy"):
    if trainer.metrics_logger.metric_exists("", name, "train"):
      h = trainer.metrics_logger.get_metric_history("", name, "train")
      print(f"{name:18s} first {h[0]:.4f}  last {h[-1]:.4f}")
  trainer.close()


if __name__ == "__main__":
  main()
