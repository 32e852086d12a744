"""Logit distillation: a small student learns from a larger teacher's output distribution.

  python examples/distillation/logit_distillation.py --steps 30

The teacher is first trained for a few steps on a synthetic next-token task (so that it knows something the student
does not), then frozen; the student minimises alpha * T^2 * KL(teacher_T || student_T) + (1 - alpha) * CE(labels).
Printed: the soft loss, the student's hard loss and the teacher's hard loss at the first and last step.
"""
from __future__ import annotations

import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch
import torch.nn.functional as F

import _common
from tunix_b200 import optim
from tunix_b200.common.configs import TrainingConfig
from tunix_b200.distillation import DistillationTrainer, TrainingInput, strategies
from tunix_b200.sft import utils as sft_utils
from tunix_b200.sft.peft_trainer import PeftTrainer, TrainingInput as SftInput

VOCAB = 96


def forward_logits(model, input_tokens, input_mask):
  positions = sft_utils.build_positions_from_mask(input_mask)
  return model(input_tokens, positions, None, sft_utils.make_causal_attn_mask(input_mask))[0]


def next_token_labels(input_tokens, input_mask):
  return F.one_hot(torch.roll(input_tokens, -1, 1), VOCAB).float()


def batches(n, batch, length, dev, cls, seed=0):
  """Sequences that count upwards from a random start (mod the vocabulary): learnable, and not trivially so."""
  g = torch.Generator().manual_seed(seed)
  for _ in range(n):
    start = torch.randint(3, VOCAB, (batch, 1), generator=g)
    ids = (3 + (start + torch.arange(length)) % (VOCAB - 3)).to(dev)
    yield cls(ids, torch.ones_like(ids))


def main() -> None:
  ap = argparse.ArgumentParser()
  ap.add_argument("--steps", type=int, default=30)
  ap.add_argument("--teacher-steps", type=int, default=30)
  ap.add_argument("--temperature", type=float, default=2.0)
  ap.add_argument("--alpha", type=float, default=0.7)
  args = ap.parse_args()
  dev = _common.device()
  teacher = _common.tiny(layers=3, width=96, vocab=VOCAB, seed=1).to(dev)
  student = _common.tiny(layers=1, width=32, vocab=VOCAB, seed=2).to(dev)
  quiet = dict(eval_every_n_steps=10**9, pbar_description=None)
  pre = PeftTrainer(teacher, optim.adamw(3e-3), TrainingConfig(max_steps=args.teacher_steps, **quiet))
  pre.train(list(batches(args.teacher_steps, 8, 32, dev, SftInput, seed=1)))
  pre.close()
  strategy = strategies.LogitStrategy(forward_logits, forward_logits, next_token_labels, temperature=args.temperature,
                                      alpha=args.alpha)
  trainer = DistillationTrainer(student, teacher, strategy, optim.adamw(3e-3), TrainingConfig(max_steps=args.steps, **quiet))
  trainer.train(list(batches(args.steps, 8, 32, dev, TrainingInput, seed=2)))
  history = lambda name: trainer.metrics_logger.get_metric_history("", name, "train")   # noqa: E731
  for name in ("distill/soft_loss", "distill/hard_loss", "distill/teacher_loss"):
    h = history(name)
    print(f"{name:22s} first {h[0]:.4f}  last {h[-1]:.4f}")
  trainer.close()


if __name__ == "__main__":
  main()
