"""Worker for the expert-parallel MoE test: 2 gloo ranks, each with its own tokens."""
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
  if a.device == "cuda":
    return main_cuda(a)
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
  # ---- optimizer step: experts in the rank-local region of the flat store, the router sharded over ranks
  from tunix_b200 import optim
  from tunix_b200.dist import fsdp
  ref2 = MoELayer(cfg)
  ref2.load_state_dict(ref.state_dict())
  ep2 = MoELayer(cfg)
  ep2.load_state_dict(ref.state_dict())
  holder2 = torch.nn.Module()
  holder2.m = ep2
  dist_moe.shard_experts(holder2, mesh)
  store = fsdp.FlatParamStore(holder2, mesh, "fsdp", transport="nccl")
  tx = optim.adamw(1e-2, weight_decay=0.1)
  state = store.init_state(tx)
  (ep2(x) ** 2).sum().backward()
  for prm in ep2.parameters():                       # autograd grads -> the store's fp32 accumulators
    if prm.grad is not None:
      prm.main_grad.add_(prm.grad)
  norm = store.step(tx, state, torch.ones(()), None)
  (ref2(x) ** 2).sum().backward()
  sq = torch.zeros(())
  worst = 0.0
  for name, prm in ref2.named_parameters():
    gsum = prm.grad.clone()
    dist.all_reduce(gsum)
    gm = gsum / world                                # denominators: 1 per rank
    sq += gm.pow(2).sum()
    new = prm.data - 1e-2 * (gm / (gm.abs() + 1e-8) + 0.1 * prm.data)
    mine = dict(ep2.named_parameters())[name].data
    want = new[sl] if name in ("gate_up_proj", "down_proj") else new
    worst = max(worst, float((mine - want).abs().max()))
  res["opt"] = worst
  res["norm"] = abs(float(norm) - float(sq.sqrt()))
  res["local_region"] = store.local_numel
  allres = [None] * world
  dist.all_gather_object(allres, res)
  if rank == 0:
    torch.save(allres, a.out)
  dist.barrier()
  dist.destroy_process_group()


def main_cuda(a):
  """2+ GPUs, NCCL for the plumbing: the peer-memory dispatch / combine with grouped tensor-core GEMMs against the
  unsharded layer (forward, input gradient, expert-weight gradient), two rounds so that buffers are reused."""
  import torch.distributed as dist
  from tunix_b200.dist import mesh as mesh_lib, moe as dist_moe
  from tunix_b200.models.transformer import ModelConfig, MoELayer
  from tunix_b200.ops import _lib
  local = int(os.environ.get("LOCAL_RANK", "0"))
  torch.cuda.set_device(local)
  dev = torch.device("cuda", local)
  mesh_lib.init_distributed("nccl", timeout_s=120)
  world, rank = dist.get_world_size(), dist.get_rank()
  mesh = mesh_lib.create_mesh((world,), ("fsdp",))
  cfg = ModelConfig(num_layers=1, vocab_size=32, embed_dim=256, hidden_dim=128, num_heads=2, head_dim=128,
                    num_kv_heads=1, num_experts=8, num_experts_per_tok=2, moe_hidden_dim=128, norm_topk_prob=True,
                    dtype=torch.bfloat16)
  torch.manual_seed(0)
  ref = MoELayer(cfg, device=dev)
  for p in ref.parameters():
    torch.nn.init.normal_(p, 0, 0.06)
  ep = MoELayer(cfg, device=dev)
  ep.load_state_dict(ref.state_dict())
  holder = torch.nn.Module()
  holder.m = ep
  dist_moe.shard_experts(holder, mesh)
  per = cfg.num_experts // world
  sl = slice(rank * per, (rank + 1) * per)
  res = {"peer": bool(dist_moe.peer_supported(ep, torch.zeros(8, 256, device=dev, dtype=torch.bfloat16)))}
  for rnd in range(2):
    g = torch.Generator().manual_seed(100 + rank + 10 * rnd)
    x = torch.randn(2, 192, 256, generator=g).to(dev, torch.bfloat16)
    xr = x.clone().requires_grad_()
    xe = x.clone().requires_grad_()
    for m in (ref, ep):
      for p in m.parameters():
        p.grad = None
    yr = ref(xr)
    ye = ep(xe)
    yr.float().pow(2).sum().backward()
    ye.float().pow(2).sum().backward()
    gref = ref.gate_up_proj.grad.float().clone()
    dist.all_reduce(gref)
    gdown = ref.down_proj.grad.float().clone()
    dist.all_reduce(gdown)
    rel = lambda a_, b_: float((a_.float() - b_.float()).abs().max() / (b_.float().abs().max() + 1e-6))
    res[f"fwd{rnd}"] = rel(ye, yr)
    res[f"dx{rnd}"] = rel(xe.grad, xr.grad)
    res[f"dw{rnd}"] = rel(ep.gate_up_proj.grad, gref[sl])
    res[f"dwd{rnd}"] = rel(ep.down_proj.grad, gdown[sl])
    gr = ref.router.w.grad.float().clone()
    res[f"drouter{rnd}"] = rel(ep.router.w.grad, gr)
  torch.cuda.synchronize()
  _lib.check_status(dev)
  allres = [None] * world
  dist.all_gather_object(allres, res)
  if rank == 0:
    torch.save(allres, a.out)
  dist.barrier()
  dist.destroy_process_group()


if __name__ == "__main__":
  main()
