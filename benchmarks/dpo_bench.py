"""DPO-with-LoRA step throughput on synthetic data (`bench.py --workload dpo`).

Qwen3-4B, LoRA rank 16 / alpha 32 on q, k, v, o, gate, up and down; the frozen reference is the
same backbone with the adapters switched off. 32 pairs per step, each a 512-token prompt with a
512-token chosen and a 512-token rejected response, sigmoid DPO with beta 0.1. Every rank trains
on its share of the pairs; adapter gradients are all-reduced.
"""
from __future__ import annotations

import json
import os
import time

import numpy as np
import torch


def run(args, ClockSampler) -> None:
  os.environ.setdefault("PYTORCH_CUDA_ALLOC_CONF", "expandable_segments:True")
  import torch.distributed as dist
  from tunix_b200 import optim
  from tunix_b200.dist import fsdp, mesh as mesh_lib
  from tunix_b200.models import automodel, dummy_model_creator, lora
  from tunix_b200.models.transformer import Transformer
  from tunix_b200.ops import _lib
  from tunix_b200.sft.dpo import dpo_trainer as dpo

  world = int(os.environ.get("WORLD_SIZE", "1"))
  rank = int(os.environ.get("RANK", "0"))
  local_rank = int(os.environ.get("LOCAL_RANK", "0"))
  torch.cuda.set_device(local_rank)
  dev = torch.device("cuda", local_rank)
  mesh = None
  if world > 1:
    mesh_lib.init_distributed("nccl")
    mesh = mesh_lib.create_mesh((world,), ("fsdp",))
    mesh_lib.set_current_mesh(mesh)
  name = args.model or "qwen3_4b"
  cfg = automodel.call_model_config(name)
  if args.layers:
    import dataclasses
    cfg = dataclasses.replace(cfg, num_layers=args.layers)
  pairs, PL, RL = args.dpo_pairs, args.dpo_prompt_len, args.dpo_response_len
  if pairs % world:
    raise SystemExit(f"{pairs} pairs do not divide over {world} ranks")
  per_rank = pairs // world
  micro = min(per_rank, args.dpo_micro)
  ga = per_rank // micro
  model = dummy_model_creator.create_dummy_model(Transformer, cfg, dtype=torch.bfloat16, device=dev, random_seed=0)
  lora.apply_lora_to_model(model, rank=16, alpha=32.0)
  with torch.no_grad():
    for n, p in model.named_parameters():
      if "lora_b" in n:
        p.normal_(0, 0.01)          # non-zero adapters so policy and reference differ
  tcfg = dpo.DPOTrainingConfig(eval_every_n_steps=10**9, gradient_accumulation_steps=ga, max_grad_norm=1.0,
                               pbar_description=None, algorithm="dpo", beta=0.1, data_sharding_axis=())
  trainer = dpo.DPOTrainer(model, dpo.ReferenceWithAdaptersOff(model), optim.adamw(1e-5, weight_decay=0.0), tcfg)
  if world > 1:
    trainer.with_grad_sync(fsdp.GradSync(model, mesh))
  trainer.is_managed_externally = True
  rng = np.random.default_rng(10 + rank)

  def batches(n_steps):
    for _ in range(n_steps * ga):
      ids = lambda n: torch.from_numpy(rng.integers(1, cfg.vocab_size - 1, size=(micro, n))).pin_memory()
      ones = lambda n: torch.ones(micro, n, dtype=torch.int32)
      yield dpo.TrainingInput(prompt_ids=ids(PL), prompt_mask=ones(PL), chosen_ids=ids(RL), chosen_mask=ones(RL),
                              rejected_ids=ids(RL), rejected_mask=ones(RL))

  def sync():
    torch.cuda.synchronize()
    if world > 1:
      dist.barrier()
      torch.cuda.synchronize()

  trainer.train(batches(args.warmup))
  sync()
  sampler = ClockSampler()
  if rank == 0:
    sampler.start()
  l0 = _lib.launch_calls
  e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
  t0 = time.perf_counter()
  e0.record()
  trainer.train(batches(args.steps))
  e1.record()
  sync()
  wall = time.perf_counter() - t0
  ms = e0.elapsed_time(e1)
  clocks = sampler.stop(local_rank) if rank == 0 else None
  _lib.check_status()
  t = torch.tensor([ms, wall], device=dev, dtype=torch.float64)
  if world > 1:
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
  ms, wall = float(t[0]), float(t[1])
  tokens = pairs * 2 * (PL + RL)
  if rank == 0:
    losses = trainer.metrics_logger.get_metric_history("", "loss", "train")
    print(json.dumps({
        "metric": "DPO (LoRA) tokens/s: policy forward+backward and reference forward over chosen and rejected rows",
        "value": tokens * args.steps / (ms / 1e3), "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic uniform token ids, random-init weights", "impl": "ours",
        "config": {"model": name, "layers": cfg.num_layers, "pairs": pairs, "prompt_len": PL, "response_len": RL,
                   "lora": "rank 16 alpha 32 on q,k,v,o,gate,up,down", "beta": 0.1, "micro_pairs": micro,
                   "grad_accum": ga, "reference": "same backbone, adapters disabled",
                   "l2": "inputs larger than L2: each pass streams the 8 GB backbone"},
        "clocks": clocks,
        "e2e": {"value": tokens * args.steps / wall, "unit": "tokens/s",
                "h2d_bytes_per_step": pairs * (PL + 2 * RL) * 8, "d2h_bytes_per_step": 8 * world},
        "gpu_launches": _lib.launch_calls - l0, "train_losses": [float(x) for x in losses],
        "peak_mem_gb": torch.cuda.max_memory_allocated() / 2**30}))
  if world > 1:
    dist.barrier()
    dist.destroy_process_group()
