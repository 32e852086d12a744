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
  # vocabulary-parallel head: log-probs and entropy from three numbers per token, full logits all-gathered
  from tunix_b200.ops import functional as Fn
  full2 = Transformer(cfg).init_weights(seed=0, scale=0.3)
  part2 = tp_lib.shard_model_tp(full2, mesh, shard_vocab=True)
  assert part2.lm_head.w.shape[0] == cfg.vocab_size // world
  got2, _ = part2(toks, pos, None, None)
  res["vp_logits"] = float((want - got2).abs().max())
  tg = torch.randint(0, 64, (2, 10))
  hf, _ = full2(toks, pos, None, None, skip_lm_head=True)
  hp, _ = part2(toks, pos, None, None, skip_lm_head=True)
  lp_f, en_f = Fn.linear_logprob(hf, full2.head_weight(), tg, temperature=0.7, want_entropy=True)
  lp_p, en_p = Fn.linear_logprob(hp, part2.head_weight(), tg, temperature=0.7, want_entropy=True)
  res["vp_logp"] = float((lp_f - lp_p).abs().max())
  res["vp_ent"] = float((en_f - en_p).abs().max())
  wgt = torch.randn(2, 10)
  ((lp_f * wgt).sum() + 0.3 * en_f.sum()).backward()
  ((lp_p * wgt).sum() + 0.3 * en_p.sum()).backward()
  f2, p2 = dict(full2.named_parameters()), dict(part2.named_parameters())
  per_v = cfg.vocab_size // world
  res["vp_dhead"] = float((f2["lm_head.w"].grad[rank * per_v:(rank + 1) * per_v] - p2["lm_head.w"].grad).abs().max())
  res["vp_dembed"] = float((f2["embedder.input_embedding"].grad - p2["embedder.input_embedding"].grad).abs().max())
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
  # vocabulary-parallel head on the kernels: per-token log-probs / entropy against the unsharded head
  from tunix_b200.ops import functional as Fn
  h = (torch.randn(48, 512, device=dev) * 0.5).to(torch.bfloat16)
  dist.broadcast(h, src=0)
  tg = torch.randint(0, 512, (48,), device=dev)
  dist.broadcast(tg, src=0)
  w_full = full.head_weight().detach().clone().requires_grad_()
  per_v = 512 // world
  w_part = w_full.detach()[rank * per_v:(rank + 1) * per_v].clone().requires_grad_()
  w_part.vocab_parallel = (mesh.group("tp"), rank * per_v)
  hf = h.clone().requires_grad_()
  hp = h.clone().requires_grad_()
  lp_f, en_f = Fn.linear_logprob(hf, w_full, tg, temperature=0.8, want_entropy=True)
  lp_p, en_p = Fn.linear_logprob(hp, w_part, tg, temperature=0.8, want_entropy=True)
  (lp_f.sum() + 0.5 * en_f.sum()).backward()
  (lp_p.sum() + 0.5 * en_p.sum()).backward()
  res["vp_logp"] = float((lp_f - lp_p).abs().max())
  res["vp_ent"] = float((en_f - en_p).abs().max())
  res["vp_dh"] = float((hf.grad.float() - hp.grad.float()).abs().max() / (hf.grad.float().abs().max() + 1e-6))
  res["vp_dw"] = float((w_full.grad.float()[rank * per_v:(rank + 1) * per_v] - w_part.grad.float()).abs().max()
                       / (w_full.grad.float().abs().max() + 1e-6))
  allres = [None] * world
  dist.all_gather_object(allres, res)
  if rank == 0:
    torch.save(allres, a.out)
  dist.barrier()
  dist.destroy_process_group()


if __name__ == "__main__":
  main()
