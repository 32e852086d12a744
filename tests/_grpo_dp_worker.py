"""Worker for the data-parallel GRPO test (launched under torchrun, gloo on CPU or NCCL on GPUs).

Every rank holds the full actor replica, rolls out its own share of the prompts with the paged
engine that shares the actor's storage, and trains with sharded optimizer state. Rank 0 writes
the final parameters and a checksum of every rank's parameters (they must agree)."""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
  ap = argparse.ArgumentParser()
  ap.add_argument("--out", required=True)
  ap.add_argument("--device", default="cpu")
  ap.add_argument("--steps", type=int, default=2)
  a = ap.parse_args()
  import torch.distributed as dist
  from tunix_b200 import optim
  from tunix_b200.common.configs import ClusterConfig, RLTrainingConfig, Role, RolloutConfig
  from tunix_b200.dist import mesh as mesh_lib
  from tunix_b200.rl import rl_cluster
  from tunix_b200.rl.grpo.grpo_learner import GRPOConfig, GRPOLearner
  from tests.test_rl_grpo import ToyTokenizer, prompts_ds, reward_len, toy_model
  from tunix_b200.ops import _lib

  world = int(os.environ.get("WORLD_SIZE", "1"))
  rank = int(os.environ.get("RANK", "0"))
  cuda = a.device == "cuda"
  mesh = None
  if world > 1:
    mesh_lib.init_distributed("nccl" if cuda else "gloo", timeout_s=120)
    mesh = mesh_lib.create_mesh((world,), ("fsdp",))
    mesh_lib.set_current_mesh(mesh)
  dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0"))) if cuda else torch.device("cpu")
  if cuda:
    torch.cuda.set_device(dev)
  if cuda:
    # large enough for every sm_100a kernel (head_dim 128 flash / paged decode, tcgen05 GEMM tiles)
    from tunix_b200.models.transformer import ModelConfig, Transformer
    mc = ModelConfig(num_layers=2, vocab_size=512, embed_dim=512, hidden_dim=1024, num_heads=4, head_dim=128,
                     num_kv_heads=2, dtype=torch.bfloat16, max_position=64)
    actor = Transformer(mc, device=dev).init_weights(seed=0, scale=0.05)
    reference = Transformer(mc, device=dev).init_weights(seed=0, scale=0.05)
  else:
    actor = toy_model(0).to(dev)
    reference = toy_model(0).to(dev)
  tc = RLTrainingConfig(actor_optimizer=optim.adamw(1e-2), eval_every_n_steps=100, max_steps=a.steps,
                        pbar_description=None, max_grad_norm=1.0)
  rc = RolloutConfig(max_tokens_to_generate=8, max_prompt_length=8, kv_cache_size=32, temperature=1.0, top_p=1.0,
                     seed=3 + rank, return_logprobs=True)
  cc = ClusterConfig(role_to_mesh={Role.ACTOR: mesh, Role.REFERENCE: mesh, Role.ROLLOUT: mesh},
                     rollout_engine="native", training_config=tc, rollout_config=rc)
  cluster = rl_cluster.RLCluster(actor=actor, reference=reference, tokenizer=ToyTokenizer(), cluster_config=cc)
  before = {n: p.detach().float().cpu().clone() for n, p in cluster.actor_trainer.model.named_parameters()}
  assert cluster.rollout.model() is cluster.actor_trainer.model       # zero-copy weight sharing
  if world > 1:
    assert hasattr(cluster.actor_trainer.model, "flat_store")
  learner = GRPOLearner(cluster, reward_fns=[reward_len], algo_config=GRPOConfig(num_generations=2, beta=0.04))
  # every rank trains on its own prompts
  batches = list(prompts_ds(a.steps * world, batch=4))[rank::world]
  learner.train(batches)
  if cuda:
    torch.cuda.synchronize()
    _lib.check_status()
  params = {n: p.detach().float().cpu() for n, p in cluster.actor_trainer.model.named_parameters()}
  moved = sum(float((params[n] - before[n]).abs().sum()) for n in params)
  checksum = torch.tensor([sum(float(p.double().sum()) for p in params.values())], dtype=torch.float64)
  sums = [checksum.clone() for _ in range(world)]
  if world > 1:
    if cuda:
      sums = [s.to(dev) for s in sums]
      dist.all_gather(sums, checksum.to(dev))
    else:
      dist.all_gather(sums, checksum)
  if rank == 0:
    torch.save({"checksums": [float(s) for s in sums], "moved": moved, "steps": cluster.global_steps,
                "loss": cluster.actor_trainer.metrics_logger.get_metric_history("", "loss", "train")}, a.out)
  if world > 1:
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
  main()
