"""Worker for the expert-parallel MoE test: 2 gloo ranks, each with its own tokens."""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
  ap = argparse.ArgumentParser()
  ap.add_argument("--out", required=True)
  a = ap.parse_args()
  import torch.distributed as dist
  from tunix_b200.dist import mesh as mesh_lib, moe as dist_moe
  from tunix_b200.models.transformer import ModelConfig, MoELayer
  mesh_lib.init_distributed("gloo", timeout_s=120)
  world, rank = dist.get_world_size(), dist.get_rank()
  mesh = mesh_lib.create_mesh((world,), ("fsdp",))
  cfg = ModelConfig(num_layers=1, vocab_size=32, embed_dim=16, hidden_dim=24, num_heads=2, head_dim=8, num_kv_heads=1,
                    num_experts=4, num_experts_per_tok=2, moe_hidden_dim=24)
  torch.manual_seed(0)
  ref = MoELayer(cfg)
  for p in ref.parameters():
    torch.nn.init.normal_(p, 0, 0.3)
  ep = MoELayer(cfg)
  ep.load_state_dict(ref.state_dict())
  holder = torch.nn.Module()
  holder.m = ep
  dist_moe.shard_experts(holder, mesh)
  g = torch.Generator().manual_seed(100 + rank)
  x = torch.randn(2, 5 + rank, 16, generator=g)          # ranks hold different numbers of tokens
  xr = x.clone().requires_grad_()
  xe = x.clone().requires_grad_()
  yr = ref(xr)
  ye = ep(xe)
  (yr ** 2).sum().backward()
  (ye ** 2).sum().backward()
  per = cfg.num_experts // world
  sl = slice(rank * per, (rank + 1) * per)
  # expert-weight gradients: the local slice of the reference gradient summed over ranks' tokens
  gref = ref.gate_up_proj.grad.clone()
  dist.all_reduce(gref)
  res = {"fwd": float((yr - ye).abs().max()), "dx": float((xr.grad - xe.grad).abs().max()),
         "dw": float((gref[sl] - ep.gate_up_proj.grad).abs().max()), "shape": tuple(ep.gate_up_proj.shape)}
  allres = [None] * world
  dist.all_gather_object(allres, res)
  if rank == 0:
    torch.save(allres, a.out)
  dist.barrier()
  dist.destroy_process_group()


if __name__ == "__main__":
  main()
