"""Worker for the sequence-parallel test: 2 gloo ranks, each holding half of every row."""
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
  from tunix_b200.dist import mesh as mesh_lib, sp as sp_lib
  from tunix_b200.models.transformer import ModelConfig, Transformer
  mesh_lib.init_distributed("gloo", timeout_s=120)
  world, rank = dist.get_world_size(), dist.get_rank()
  mesh = mesh_lib.create_mesh((world,), ("sp",))
  cfg = ModelConfig(num_layers=2, vocab_size=64, embed_dim=32, hidden_dim=48, num_heads=4, head_dim=8, num_kv_heads=2,
                    use_qk_norm=True)
  full = Transformer(cfg).init_weights(seed=3, scale=0.2)
  part = Transformer(cfg).init_weights(seed=3, scale=0.2)
  sp_lib.shard_model_sp(part, mesh, "sp")
  g = torch.Generator().manual_seed(7)
  tokens = torch.randint(0, 64, (2, 12), generator=g)
  target = torch.randn(2, 12, 64, generator=g)
  logits_full, _ = full(tokens, torch.arange(12)[None].expand(2, 12), None, None)
  (logits_full * target).sum().backward()
  mine, pos = sp_lib.local_chunk(tokens, mesh, "sp")
  T = mine.shape[1]
  logits_part, _ = part(mine, pos, None, None)
  (logits_part * target[:, rank * T:(rank + 1) * T]).sum().backward()
  sp_lib.reduce_gradients(part, mesh.group("sp"))
  res = {"fwd": float((logits_part - logits_full[:, rank * T:(rank + 1) * T]).abs().max()), "grads": 0.0}
  fp = dict(full.named_parameters())
  for n, p in part.named_parameters():
    if p.grad is None:
      continue
    res["grads"] = max(res["grads"], float((p.grad - fp[n].grad).abs().max()))
  allres = [None] * world
  dist.all_gather_object(allres, res)
  if rank == 0:
    torch.save(allres, a.out)
  dist.barrier()
  dist.destroy_process_group()


if __name__ == "__main__":
  main()
