"""Worker for the tensor-parallel test: 2 gloo ranks hold half the heads / hidden units each."""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
  ap = argparse.ArgumentParser()
  ap.add_argument("--out", required=True)
  ap.add_argument("--device", default="cpu")
  a = ap.parse_args()
  import torch.distributed as dist
  from tunix_b200.dist import mesh as mesh_lib, tp as tp_lib
  from tunix_b200.models.transformer import ModelConfig, Transformer
  if a.device == "cuda":
    return main_cuda(a)
  mesh_lib.init_distributed("gloo", timeout_s=120)
  world, rank = dist.get_world_size(), dist.get_rank()
  mesh = mesh_lib.create_mesh((world,), ("tp",))
  cfg = ModelConfig(num_layers=2, vocab_size=64, embed_dim=32, hidden_dim=48, num_heads=4, head_dim=8, num_kv_heads=2,
                    use_qk_norm=True)
  full = Transformer(cfg).init_weights(seed=0, scale=0.3)
  part = tp_lib.shard_model_tp(full, mesh)
  assert part.config.num_heads == 2 and part.config.num_kv_heads == 1 and part.config.hidden_dim == 24
  torch.manual_seed(5)
  toks = torch.randint(0, 64, (2, 10))
  pos = torch.arange(10)[None].expand(2, 10)
  want, _ = full(toks, pos, None, None)
  got, _ = part(toks, pos, None, None)
  (want.float() ** 2).mean().backward()
  (got.float() ** 2).mean().backward()
  fp, pp = dict(full.named_parameters()), dict(part.named_parameters())
  res = {"fwd": float((want - got).abs().max()),
         "d_embed": float((fp["embedder.input_embedding"].grad - pp["embedder.input_embedding"].grad).abs().max()),
         "d_norm": float((fp["layers.0.input_layernorm.w"].grad - pp["layers.0.input_layernorm.w"].grad).abs().max())}
  # a sharded weight's gradient is the matching slice of the full gradient
  per = cfg.hidden_dim // world
  gfull = fp["layers.1.mlp.down_proj.w"].grad[:, rank * per:(rank + 1) * per]
  res["d_down"] = float((gfull - pp["layers.1.mlp.down_proj.inner.w"].grad).abs().max())
  # decoding with a KV cache works on the slice too (fewer kv heads per rank)
  from tunix_b200.generate import utils as gen_utils  # noqa: F401
  allres = [None] * world
  dist.all_gather_object(allres, res)
  if rank == 0:
    torch.save(allres, a.out)
  dist.barrier()
  dist.destroy_process_group()


def main_cuda(a):
  """2 GPUs: the row-parallel exits run the GEMM with the all-reduce epilogue over peer memory."""
  import torch.distributed as dist
  from tunix_b200.dist import mesh as mesh_lib, tp as tp_lib
  from tunix_b200.models.transformer import ModelConfig, Transformer
  from tunix_b200.ops import _lib
  local = int(os.environ.get("LOCAL_RANK", "0"))
  torch.cuda.set_device(local)
  dev = torch.device("cuda", local)
  mesh_lib.init_distributed("nccl", timeout_s=120)
  world, rank = dist.get_world_size(), dist.get_rank()
  mesh = mesh_lib.create_mesh((world,), ("tp",))
  cfg = ModelConfig(num_layers=2, vocab_size=512, embed_dim=512, hidden_dim=1024, num_heads=4, head_dim=128,
                    num_kv_heads=2, dtype=torch.bfloat16, max_position=64)
  full = Transformer(cfg, device=dev).init_weights(seed=0, scale=0.05)
  part = tp_lib.shard_model_tp(full, mesh, fused_max_rows=64)
  assert isinstance(part.layers[0].attn.o_proj, tp_lib.FusedRowExit)
  torch.manual_seed(5)
  res = {}
  with torch.no_grad():
    for i, L in enumerate((16, 32, 8)):                  # repeated calls reuse the sum buffers
      toks = torch.randint(0, 512, (2, L), device=dev)
      pos = torch.arange(L, device=dev)[None].expand(2, L)
      want, _ = full(toks, pos, None, None)
      got, _ = part(toks, pos, None, None)
      res[f"fwd{i}"] = float((want.float() - got.float()).abs().max() / want.float().abs().max())
  torch.cuda.synchronize()
  _lib.check_status()
  # with gradients enabled the exits fall back to GEMM + all-reduce
  toks = torch.randint(0, 512, (2, 16), device=dev)
  pos = torch.arange(16, device=dev)[None].expand(2, 16)
  got, _ = part(toks, pos, None, None)
  got.float().pow(2).mean().backward()
  res["grad_ok"] = all(p.grad is not None for n, p in part.named_parameters() if "inner.w" in n)
  allres = [None] * world
  dist.all_gather_object(allres, res)
  if rank == 0:
    torch.save(allres, a.out)
  dist.barrier()
  dist.destroy_process_group()


if __name__ == "__main__":
  main()
