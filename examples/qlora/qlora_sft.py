"""QLoRA: the frozen projections are stored in NF4 (4 bits per weight plus per-tile scales), adapters train in the
compute dtype.

  python examples/qlora/qlora_sft.py --steps 20
  python examples/qlora/qlora_sft.py --model llama3p2_1b --rank 16 --steps 100        # on a GPU

Printed: bytes held by the adapted projections before and after quantisation, the number of trainable parameters,
and the loss at the first and last step.
"""
from __future__ import annotations

import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch

import _common
from tunix_b200 import optim
from tunix_b200.common.configs import TrainingConfig
from tunix_b200.models import lora as lora_lib
from tunix_b200.models.transformer import Linear, Transformer
from tunix_b200.sft.peft_trainer import PeftTrainer, TrainingInput


def projection_bytes(model) -> int:
  total = 0
  for mod in model.modules():
    if isinstance(mod, Linear):
      total += sum(t.numel() * t.element_size() for t in mod.state_dict().values() if isinstance(t, torch.Tensor))
  return total


def main() -> None:
  ap = argparse.ArgumentParser()
  ap.add_argument("--model", default="tiny")
  ap.add_argument("--steps", type=int, default=20)
  ap.add_argument("--rank", type=int, default=8)
  ap.add_argument("--tile-size", type=int, default=64)
  args = ap.parse_args()
  dev = _common.device()
  if args.model == "tiny":
    model = _common.tiny(layers=2, width=128, vocab=160)
  else:
    from tunix_b200.models.llama3 import model as llama
    model = Transformer(getattr(llama.ModelConfig, args.model)()).init_weights(seed=0)
  model = model.to(dev, torch.bfloat16 if dev.type == "cuda" else torch.float32)
  before = projection_bytes(model)
  lora_lib.apply_lora_to_model(model, rank=args.rank, alpha=2.0 * args.rank, weight_qtype="nf4", tile_size=args.tile_size)
  after = projection_bytes(model)
  trainable = sum(p.numel() for p in model.parameters() if p.requires_grad)
  print(f"projections: {before / 2**20:.2f} MiB -> {after / 2**20:.2f} MiB with NF4 weights and rank-{args.rank} adapters; "
        f"{trainable:,d} trainable parameters")
  g = torch.Generator().manual_seed(0)
  vocab = model.config.vocab_size
  data = []
  for _ in range(args.steps):
    start = torch.randint(3, vocab, (4, 1), generator=g)
    ids = (3 + (start + 2 * torch.arange(48)) % (vocab - 3)).to(dev)
    data.append(TrainingInput(ids, torch.ones_like(ids)))
  trainer = PeftTrainer(model, optim.adamw(5e-3), TrainingConfig(max_steps=args.steps, eval_every_n_steps=10**9,
                                                                  pbar_description=None))
  trainer.train(data)
  losses = trainer.metrics_logger.get_metric_history("", "loss", "train")
  print(f"loss: first {losses[0]:.4f}  last {losses[-1]:.4f}")
  trainer.close()


if __name__ == "__main__":
  main()
