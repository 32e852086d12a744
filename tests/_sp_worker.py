"""Worker for the sequence-parallel tests: each rank holds its chunks of every row. gloo ranks on CPU in fp32,
or NCCL ranks on GPUs in bf16 (keys and values pulled through peer-mapped buffers)."""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
  ap = argparse.ArgumentParser()
  ap.add_argument("--out", required=True)
  ap.add_argument("--layout", default="contiguous")
  ap.add_argument("--backend", default="gloo")
  a = ap.parse_args()
  import torch.distributed as dist
  from tunix_b200.dist import mesh as mesh_lib, sp as sp_lib
  from tunix_b200.models.transformer import ModelConfig, Transformer
  gpu = a.backend == "nccl"
  if gpu:
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
  mesh_lib.init_distributed(a.backend, timeout_s=120)
  world, rank = dist.get_world_size(), dist.get_rank()
  mesh = mesh_lib.create_mesh((world,), ("sp",))
  if gpu:     # shapes the flash kernels take: head_dim 128, chunks of 256 tokens
    cfg = ModelConfig(num_layers=2, vocab_size=512, embed_dim=256, hidden_dim=512, num_heads=4, head_dim=128,
                      num_kv_heads=2, use_qk_norm=True)
    V, L, dev, dt, scale = 512, 1024, torch.device("cuda"), torch.bfloat16, 0.05
  else:
    cfg = ModelConfig(num_layers=2, vocab_size=64, embed_dim=32, hidden_dim=48, num_heads=4, head_dim=8,
                      num_kv_heads=2, use_qk_norm=True)
    V, L, dev, dt, scale = 64, 12, torch.device("cpu"), torch.float32, 0.2
  full = Transformer(cfg).init_weights(seed=3, scale=scale).to(dev, dt)
  part = Transformer(cfg).init_weights(seed=3, scale=scale).to(dev, dt)
  sp_lib.shard_model_sp(part, mesh, "sp", layout=a.layout)
  g = torch.Generator().manual_seed(7)
  tokens = torch.randint(0, V, (2, L), generator=g).to(dev)
  target = torch.randn(2, L, V, generator=g).to(dev, dt)
  logits_full, _ = full(tokens, torch.arange(L, device=dev)[None].expand(2, L), None, None)
  (logits_full * target).sum().backward()
  mine, pos = sp_lib.local_chunk(tokens, mesh, "sp", layout=a.layout)
  logits_part, _ = part(mine, pos, None, None)
  (logits_part * sp_lib.local_rows(target, mesh, "sp", layout=a.layout)).sum().backward()
  sp_lib.reduce_gradients(part, mesh.group("sp"))
  want = sp_lib.local_rows(logits_full, mesh, "sp", layout=a.layout)
  fp = dict(full.named_parameters())
  if gpu:     # bf16: errors relative to the size of what is compared
    from tunix_b200.ops import _lib
    _lib.check_status(dev)
    res = {"fwd": float((logits_part.float() - want.float()).norm() / want.float().norm()), "grads": 0.0}
    for n, p in part.named_parameters():
      if p.grad is not None:
        ref = fp[n].grad.float()
        res["grads"] = max(res["grads"], float((p.grad.float() - ref).norm() / (ref.norm() + 1e-6)))
  else:
    res = {"fwd": float((logits_part - want).abs().max()), "grads": 0.0}
    for n, p in part.named_parameters():
      if p.grad is not None:
        res["grads"] = max(res["grads"], float((p.grad - fp[n].grad).abs().max()))
  allres = [None] * world
  dist.all_gather_object(allres, res)
  if rank == 0:
    torch.save(allres, a.out)
  dist.barrier()
  dist.destroy_process_group()


if __name__ == "__main__":
  main()
