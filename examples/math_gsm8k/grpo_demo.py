"""Single-turn GRPO on arithmetic word problems (the GSM8K demo of the reference, with synthetic problems).

  python examples/math_gsm8k/grpo_demo.py --steps 4                                  # tiny random model on CPU
  python examples/math_gsm8k/grpo_demo.py --model qwen3_0p6b --steps 50               # one GPU
  torchrun --nproc-per-node 8 --master-addr 127.0.0.1 examples/math_gsm8k/grpo_demo.py \\
      --model qwen3_8b --rollout-tp 2                                                  # FSDP trainer, TP-2 rollout

Rewards: +1 for a correct final number, +0.25 for an answer in the expected format.
"""
from __future__ import annotations

import argparse
import os
import re
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

import torch

from tunix_b200 import optim
from tunix_b200.common.configs import ClusterConfig, RLTrainingConfig, RolloutConfig
from tunix_b200.common.datatypes import Role
from tunix_b200.dist import mesh as mesh_lib
from tunix_b200.examples.data import math_dataset
from tunix_b200.models.qwen3 import model as qwen3
from tunix_b200.models.transformer import ModelConfig, Transformer
from tunix_b200.rl import rl_cluster
from tunix_b200.rl.grpo import grpo_learner

_NUMBER = re.compile(r"-?\d+(?:\.\d+)?")


class DigitTokenizer:
  """Characters as tokens (digits, letters, punctuation): small vocabulary, exact round trip."""

  def __init__(self):
    self.chars = [chr(c) for c in range(32, 127)]

  def encode(self, text, **_):
    return [3 + self.chars.index(c) for c in text if c in self.chars]

  def decode(self, ids, **_):
    return "".join(self.chars[i - 3] for i in ids if 3 <= i < 3 + len(self.chars))

  def bos_id(self):
    return 1

  def eos_id(self):
    return 2

  def pad_id(self):
    return 0


def correct_answer(prompts, completions, answer=None, **_):
  scores = []
  for text, want in zip(completions, answer):
    found = _NUMBER.findall(text)
    scores.append(1.0 if found and abs(float(found[-1]) - float(want)) < 1e-6 else 0.0)
  return scores


def answer_format(prompts, completions, **_):
  return [0.25 if _NUMBER.search(text) else 0.0 for text in completions]


def batches(n, batch):
  ds = math_dataset.create_dataset("synthetic", as_messages=False, num_synthetic=n * batch)
  for i in range(n):
    rows = [ds[i * batch + j] for j in range(batch)]
    yield {"prompts": [r["prompts"] for r in rows], "answer": [r["answer"] for r in rows]}


def main() -> None:
  ap = argparse.ArgumentParser()
  ap.add_argument("--model", default="tiny")
  ap.add_argument("--steps", type=int, default=4)
  ap.add_argument("--prompts", type=int, default=4, help="prompts per step (per rank)")
  ap.add_argument("--generations", type=int, default=4)
  ap.add_argument("--new-tokens", type=int, default=16)
  ap.add_argument("--rollout-tp", type=int, default=1)
  ap.add_argument("--beta", type=float, default=0.0)
  args = ap.parse_args()

  world = int(os.environ.get("WORLD_SIZE", "1"))
  cuda = torch.cuda.is_available()
  dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0"))) if cuda else torch.device("cpu")
  mesh = None
  if world > 1:
    mesh_lib.init_distributed()
    mesh = mesh_lib.create_mesh((world,), ("fsdp",))
    mesh_lib.set_current_mesh(mesh)
  tok = DigitTokenizer()
  if args.model == "tiny":
    cfg = ModelConfig(num_layers=2, vocab_size=128, embed_dim=64, hidden_dim=128, num_heads=4, head_dim=16, num_kv_heads=2)
  else:
    cfg = getattr(qwen3.ModelConfig, args.model)()
  dtype = torch.bfloat16 if cuda else torch.float32
  actor = Transformer(cfg).init_weights(seed=0, scale=0.05).to(dev, dtype)
  reference = Transformer(cfg).init_weights(seed=0, scale=0.05).to(dev, dtype) if args.beta else None
  tc = RLTrainingConfig(actor_optimizer=optim.adamw(1e-5 if args.model != "tiny" else 1e-3), eval_every_n_steps=10**6,
                        max_steps=args.steps, pbar_description=None)
  rc = RolloutConfig(max_tokens_to_generate=args.new_tokens, max_prompt_length=640, kv_cache_size=640 + args.new_tokens + 8,
                     temperature=1.0, top_p=1.0, return_logprobs=True, tensor_parallel_size=args.rollout_tp)
  cc = ClusterConfig(role_to_mesh={Role.ACTOR: mesh, Role.REFERENCE: mesh, Role.ROLLOUT: mesh},
                     rollout_engine="native" if cuda else "vanilla", training_config=tc, rollout_config=rc)
  cluster = rl_cluster.RLCluster(actor=actor, reference=reference, tokenizer=tok, cluster_config=cc)
  learner = grpo_learner.GRPOLearner(
      rl_cluster=cluster, reward_fns=[correct_answer, answer_format],
      algo_config=grpo_learner.GRPOConfig(num_generations=args.generations, beta=args.beta or None))
  learner.train(batches(args.steps, args.prompts))
  if int(os.environ.get("RANK", "0")) == 0:
    print(f"optimizer steps {cluster.actor_trainer.train_steps}, weight sync {cluster.weight_sync_ms()} ms")


if __name__ == "__main__":
  main()
