"""Supervised fine-tuning on synthetic translation pairs.

  python examples/sft/sft_synthetic.py --steps 20                 # tiny random model, CPU or one GPU
  python examples/sft/sft_synthetic.py --model llama3p2_1b --lora-rank 16 --steps 100
  torchrun --nproc-per-node 8 --master-addr 127.0.0.1 examples/sft/sft_synthetic.py --model llama3p1_8b
"""
from __future__ import annotations

import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

import torch

from tunix_b200 import optim
from tunix_b200.common.configs import TrainingConfig
from tunix_b200.dist import mesh as mesh_lib
from tunix_b200.examples.data import translation_dataset
from tunix_b200.models import lora as lora_lib
from tunix_b200.models.llama3 import model as llama
from tunix_b200.models.transformer import ModelConfig, Transformer
from tunix_b200.sft.peft_trainer import PeftTrainer


class WordTokenizer:
  """Whitespace tokenizer over a growing vocabulary: enough for synthetic data, no files needed."""

  def __init__(self, size: int):
    self.size, self.ids = size, {}

  def encode(self, text, **_):
    return [self.ids.setdefault(w, 3 + len(self.ids) % (self.size - 3)) for w in text.split()]

  def tokenize(self, example, prefix="", suffix="", add_eos=True):
    import numpy as np
    ids = [self.bos_id()] + self.encode(prefix + example + suffix) + ([self.eos_id()] if add_eos else [])
    return np.asarray(ids, dtype=np.int32)

  def decode(self, ids, **_):
    return " ".join(str(i) for i in ids)

  def bos_id(self):
    return 1

  def eos_id(self):
    return 2

  def pad_id(self):
    return 0


def main() -> None:
  ap = argparse.ArgumentParser()
  ap.add_argument("--model", default="tiny", help="tiny, or a preset of models.llama3 (llama3p2_1b, llama3p1_8b, ...)")
  ap.add_argument("--steps", type=int, default=20)
  ap.add_argument("--batch", type=int, default=8)
  ap.add_argument("--seq-len", type=int, default=64)
  ap.add_argument("--lora-rank", type=int, default=0)
  ap.add_argument("--lr", type=float, default=1e-3)
  ap.add_argument("--checkpoint-dir", default="")
  args = ap.parse_args()

  world = int(os.environ.get("WORLD_SIZE", "1"))
  dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0"))) if torch.cuda.is_available() else torch.device("cpu")
  mesh = None
  if world > 1:
    mesh_lib.init_distributed()
    mesh = mesh_lib.create_mesh((world,), ("fsdp",))
    mesh_lib.set_current_mesh(mesh)
  if args.model == "tiny":
    cfg = ModelConfig(num_layers=2, vocab_size=512, embed_dim=64, hidden_dim=128, num_heads=4, head_dim=16, num_kv_heads=2)
  else:
    cfg = getattr(llama.ModelConfig, args.model)()
  dtype = torch.bfloat16 if dev.type == "cuda" else torch.float32
  model = Transformer(cfg).init_weights(seed=0).to(dev, dtype)
  if args.lora_rank:
    lora_lib.apply_lora_to_model(model, rank=args.lora_rank, alpha=2.0 * args.lora_rank)
  if mesh is not None or dev.type == "cuda":
    from tunix_b200.dist import fsdp
    model = fsdp.shard_model(model, mesh)     # flat bf16 parameters, fp32 gradients, optimizer state sharded over the mesh
  tok = WordTokenizer(cfg.vocab_size)
  train, evald = translation_dataset.create_datasets("synthetic", args.batch, args.seq_len, None, tok)
  trainer = PeftTrainer(model, optim.adamw(args.lr), TrainingConfig(
      eval_every_n_steps=max(1, args.steps // 2), max_steps=args.steps,
      checkpoint_root_directory=args.checkpoint_dir or None, pbar_description=None))
  trainer.train(train, evald)
  losses = trainer.metrics_logger.get_metric_history("", "loss", "train")
  if int(os.environ.get("RANK", "0")) == 0:
    print(f"steps {len(losses)}  first loss {losses[0]:.4f}  last loss {losses[-1]:.4f}")
  trainer.close()


if __name__ == "__main__":
  main()
