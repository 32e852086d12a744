"""Library baseline for the headline benchmark: the same Llama-3.1-8B SFT step written with stock
PyTorch only - `torch.nn.functional` ops (cuBLAS GEMMs, library scaled-dot-product attention),
`torch.distributed.fsdp.fully_shard` (NCCL all-gather / reduce-scatter) and `torch.optim.AdamW`.
None of this repository's kernels, engine or models are imported. It is the "NCCL + cuBLAS"
arm that the fused sm_100a build is compared with when the JAX reference cannot be installed.

Numerics match the headline configuration: fp32 master weights and AdamW state, bf16 compute
(FSDP mixed precision: parameters are cast to bf16 for forward / backward, gradients are reduced
in fp32), global-norm clipping at 1.0, loss on all tokens, activation checkpointing per layer.
"""
from __future__ import annotations

import json
import math
import os
import time

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F
from torch.utils.checkpoint import checkpoint

CONFIGS = {
    "llama3p1_8b": dict(layers=32, dim=4096, heads=32, kv_heads=8, head_dim=128, ffn=14336, vocab=128256,
                        theta=500000.0, eps=1e-5),
}


def rope_tables(seq: int, head_dim: int, theta: float, device):
  inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, device=device, dtype=torch.float32) / head_dim))
  ang = torch.arange(seq, device=device, dtype=torch.float32)[:, None] * inv[None]
  return ang.cos(), ang.sin()


def apply_rope(x, cos, sin):
  # x [B, T, N, H]; half-split rotation
  x1, x2 = x.float().chunk(2, dim=-1)
  c, s = cos[None, :, None, :], sin[None, :, None, :]
  return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1).to(x.dtype)


class Block(nn.Module):
  def __init__(self, c):
    super().__init__()
    D, N, K, H, Fh = c["dim"], c["heads"], c["kv_heads"], c["head_dim"], c["ffn"]
    self.c = c
    self.ln1 = nn.Parameter(torch.ones(D))
    self.ln2 = nn.Parameter(torch.ones(D))
    self.qkv = nn.Linear(D, (N + 2 * K) * H, bias=False)
    self.o = nn.Linear(N * H, D, bias=False)
    self.gate_up = nn.Linear(D, 2 * Fh, bias=False)
    self.down = nn.Linear(Fh, D, bias=False)

  def forward(self, h, cos, sin):
    c = self.c
    N, K, H = c["heads"], c["kv_heads"], c["head_dim"]
    B, T, D = h.shape
    x = F.rms_norm(h, (D,), self.ln1.to(h.dtype), c["eps"])
    q, k, v = self.qkv(x).split([N * H, K * H, K * H], dim=-1)
    q = apply_rope(q.view(B, T, N, H), cos, sin).transpose(1, 2)
    k = apply_rope(k.view(B, T, K, H), cos, sin).transpose(1, 2)
    v = v.view(B, T, K, H).transpose(1, 2)
    a = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True)
    h = h + self.o(a.transpose(1, 2).reshape(B, T, N * H))
    x = F.rms_norm(h, (D,), self.ln2.to(h.dtype), c["eps"])
    g, u = self.gate_up(x).chunk(2, dim=-1)
    return h + self.down(F.silu(g) * u)


class Llama(nn.Module):
  def __init__(self, c):
    super().__init__()
    self.c = c
    self.embed = nn.Embedding(c["vocab"], c["dim"])
    self.blocks = nn.ModuleList([Block(c) for _ in range(c["layers"])])
    self.norm = nn.Parameter(torch.ones(c["dim"]))
    self.head = nn.Linear(c["dim"], c["vocab"], bias=False)

  def forward(self, tokens, cos, sin, targets):
    """Sum of the token cross-entropies (the head runs inside the module, where its weight is gathered)."""
    h = self.embed(tokens)
    for b in self.blocks:
      h = checkpoint(b, h, cos, sin, use_reentrant=False)
    h = F.rms_norm(h, (self.c["dim"],), self.norm.to(h.dtype), self.c["eps"])
    return chunked_loss(h.reshape(-1, self.c["dim"]), self.head.weight, targets.reshape(-1))


def chunked_loss(hidden, head_w, targets, chunk=2048):
  """Sum of token cross-entropies with the [T, V] logits materialised one chunk at a time."""
  T = hidden.shape[0]
  total = hidden.new_zeros((), dtype=torch.float32)
  for s in range(0, T, chunk):
    def f(hc, tc):
      return F.cross_entropy(F.linear(hc, head_w).float(), tc, reduction="sum")
    total = total + checkpoint(f, hidden[s:s + chunk], targets[s:s + chunk], use_reentrant=False)
  return total


def run(args, clock_sampler_cls) -> None:
  from torch.distributed.fsdp import MixedPrecisionPolicy, fully_shard
  world = int(os.environ.get("WORLD_SIZE", "1"))
  rank = int(os.environ.get("RANK", "0"))
  local = int(os.environ.get("LOCAL_RANK", "0"))
  torch.cuda.set_device(local)
  dev = torch.device("cuda", local)
  if not dist.is_initialized():      # fully_shard needs a process group, also for one rank
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29599")
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
  c = dict(CONFIGS[args.model or "llama3p1_8b"])
  if args.layers:
    c["layers"] = args.layers
  S, GB = args.seq_len, args.global_batch or 64
  micro = args.micro_batch or 1
  per_gpu = GB // world
  ga = per_gpu // micro
  torch.manual_seed(1234)
  with torch.device("meta"):
    model = Llama(c)
  mp = MixedPrecisionPolicy(param_dtype=torch.bfloat16, reduce_dtype=torch.float32)
  for b in model.blocks:
    fully_shard(b, mp_policy=mp)
  fully_shard(model, mp_policy=mp)
  model.to_empty(device=dev)
  with torch.no_grad():
    for p in model.parameters():
      if p.dim() > 1:
        p.normal_(0.0, 0.02)
      else:
        p.fill_(1.0)
  opt = torch.optim.AdamW(model.parameters(), lr=1e-5, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, fused=True)
  cos, sin = rope_tables(S, c["head_dim"], c["theta"], dev)
  g = torch.Generator().manual_seed(1000 + rank)
  host = [torch.randint(0, c["vocab"], (micro, S), generator=g, dtype=torch.int32).pin_memory() for _ in range(2 * ga)]
  resident = [t.to(dev).long() for t in host]
  losses = []

  def step(batches, from_host: bool):
    total = torch.zeros((), device=dev)
    for i, tok in enumerate(batches):
      if from_host:
        tok = tok.to(dev, non_blocking=True).long()
      model.set_requires_gradient_sync(i == len(batches) - 1)       # reduce-scatter once per optimizer step
      loss = model(tok[:, :-1], cos[:S - 1], sin[:S - 1], tok[:, 1:])
      (loss / (GB * (S - 1))).backward()
      total += loss.detach()
    torch.nn.utils.clip_grad_norm_(model.parameters(), 1.0)
    opt.step()
    opt.zero_grad(set_to_none=True)
    return total / (per_gpu * (S - 1))

  def sync():
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()

  def batch_list(k):
    return [resident[(k * ga + i) % len(resident)] for i in range(ga)]

  for k in range(args.warmup):
    losses.append(float(step(batch_list(k), False)))
  sync()
  sampler = clock_sampler_cls()
  if rank == 0:
    sampler.start()
  e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
  e0.record()
  step_losses = [step(batch_list(args.warmup + k), False) for k in range(args.steps)]
  e1.record()
  sync()
  ms = e0.elapsed_time(e1)
  clocks = sampler.stop(local) if rank == 0 else None
  losses += [float(x) for x in step_losses]
  t = torch.tensor([ms], device=dev)
  dist.all_reduce(t, op=dist.ReduceOp.MAX)
  ms = float(t.item())
  tokens_per_step = GB * S
  e2e = None
  if not args.no_e2e:
    step([host[i % len(host)] for i in range(ga)], True)
    sync()
    t0 = time.perf_counter()
    e2e_losses = []
    for k in range(args.steps):
      e2e_losses.append(float(step([host[(k * ga + i) % len(host)] for i in range(ga)], True)))   # D2H read of the loss
    torch.cuda.synchronize()
    dt = torch.tensor([time.perf_counter() - t0], device=dev)
    dist.all_reduce(dt, op=dist.ReduceOp.MAX)
    e2e = {"value": tokens_per_step * args.steps / float(dt.item()), "unit": "tokens/s",
           "h2d_bytes_per_step": GB * S * 4, "d2h_bytes_per_step": 4 * world, "losses": e2e_losses}
  if rank == 0:
    nparams = sum(p.numel() for p in model.parameters()) * 1  # sharded parameters report their global size
    out = {"metric": "SFT tokens/s (Llama-3.1-8B full-weight, bf16 + fp32 master AdamW, seq 4096, global batch 64)",
           "value": tokens_per_step * args.steps / (ms / 1e3), "unit": "tokens/s", "n_gpus": world,
           "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
           "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
           "data": "synthetic uniform token ids, random-init N(0,0.02) weights", "impl": "torch_baseline",
           "config": {"model": args.model or "llama3p1_8b", "layers": c["layers"], "global_batch": GB, "seq_len": S,
                      "parallelism": f"torch fully_shard x{world} (NCCL), cuBLAS GEMMs, library SDPA, fused AdamW",
                      "micro_batch_per_gpu": micro, "grad_accum": ga, "remat": "per layer",
                      "l2": "inputs larger than L2: each step streams >100 GB of weights, gradients and optimizer state",
                      "optimizer": "AdamW fp32 params/m/v, global-norm clip 1.0"},
           "clocks": clocks, "e2e": e2e, "gpu_launches": 0, "train_losses": losses, "parameters": nparams,
           "peak_mem_gb": torch.cuda.max_memory_allocated() / 2 ** 30}
    print(json.dumps(out))
  dist.barrier()
  dist.destroy_process_group()
