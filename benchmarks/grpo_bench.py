"""GRPO step throughput on synthetic data (the second headline workload of `bench.py`).

Qwen3-8B, 64 prompts of 256 uniform-random tokens x G=8 samples, up to 768 new tokens at
temperature 1, reward = fraction of generated ids divisible by 7, KL beta 0.04 against a frozen
reference, clip 0.2, one policy update per batch. Every rank keeps a resident bf16 replica of
the actor, so rollout is data-parallel over ranks on the same storage the trainer updates
(no weight copy between trainer and rollout) and the optimizer state is sharded.

A step = rollout + reference log-probs + policy update. Timed on the device with CUDA events
around K steps after W warm-up steps, max over ranks.
"""
from __future__ import annotations

import json
import os
import time
from typing import List

import numpy as np
import torch


class IntTokenizer:
  """Text is a space-separated list of token ids, so synthetic id sequences survive the string API."""

  def __init__(self, vocab: int):
    self.vocab = vocab

  def encode(self, s, **kw):
    return [int(w) for w in s.split()]

  def decode(self, ids, **kw):
    return " ".join(str(int(i)) for i in ids)

  def bos_id(self): return None
  def eos_id(self): return self.vocab - 1
  def pad_id(self): return 0


def reward_mod7(prompts, completions, **kw) -> List[float]:
  out = []
  for c in completions:
    ids = c.split()
    out.append(sum(1 for w in ids if int(w) % 7 == 0) / max(len(ids), 1))
  return out


def run(args, ClockSampler) -> None:
  os.environ.setdefault("PYTORCH_CUDA_ALLOC_CONF", "expandable_segments:True")
  import torch.distributed as dist
  from tunix_b200 import optim
  from tunix_b200.common.configs import ClusterConfig, RLTrainingConfig, Role, RolloutConfig
  from tunix_b200.dist import mesh as mesh_lib
  from tunix_b200.models import automodel, dummy_model_creator
  from tunix_b200.models.transformer import Transformer
  from tunix_b200.ops import _lib
  from tunix_b200.rl import rl_cluster
  from tunix_b200.rl.grpo.grpo_learner import GRPOConfig, GRPOLearner
  from tunix_b200.rl.rollout import native_rollout

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

  model_name = args.model or "qwen3_8b"
  cfg = automodel.call_model_config(model_name)
  if args.layers:
    import dataclasses
    cfg = dataclasses.replace(cfg, num_layers=args.layers)
  P, G, NEW, PL = args.grpo_prompts, args.grpo_generations, args.grpo_new_tokens, args.grpo_prompt_len
  if P % world:
    raise SystemExit(f"{P} prompts do not divide over {world} ranks")
  per_rank = P // world
  actor = dummy_model_creator.create_dummy_model(Transformer, cfg, dtype=torch.bfloat16, device=dev, random_seed=0)
  reference = dummy_model_creator.create_dummy_model(Transformer, cfg, dtype=torch.bfloat16, device=dev, random_seed=0)
  for p in reference.parameters():
    p.requires_grad_(False)
  tok = IntTokenizer(cfg.vocab_size)
  steps_total = args.warmup + args.steps
  tc = RLTrainingConfig(actor_optimizer=optim.adamw(1e-6, b1=0.9, b2=0.95, weight_decay=0.1),
                        eval_every_n_steps=10**9, max_steps=steps_total, pbar_description=None, max_grad_norm=1.0,
                        mini_batch_size=per_rank, train_micro_batch_size=args.grpo_train_micro,
                        rollout_micro_batch_size=per_rank, compute_logps_micro_batch_size=args.grpo_train_micro)
  tp = max(1, int(getattr(args, "rollout_tp", 1)))
  if world % tp:
    raise SystemExit(f"--rollout-tp {tp} does not divide {world} GPUs")
  # the ranks of a tensor-parallel rollout group decode one batch together: they must draw with one seed
  rc = RolloutConfig(max_tokens_to_generate=NEW, max_prompt_length=PL, kv_cache_size=PL + NEW + 16,
                     temperature=1.0, top_p=1.0, seed=1000 + rank // tp, return_logprobs=True,
                     tensor_parallel_size=tp if tp > 1 else -1, data_parallel_size=world // tp if tp > 1 else -1)
  cc = ClusterConfig(role_to_mesh={Role.ACTOR: mesh, Role.REFERENCE: mesh, Role.ROLLOUT: mesh},
                     rollout_engine="native", training_config=tc, rollout_config=rc)
  native_rollout.DEFAULT_MAX_BATCH = args.grpo_rollout_batch
  cluster = rl_cluster.RLCluster(actor=actor, reference=reference, tokenizer=tok, cluster_config=cc)
  learner = GRPOLearner(cluster, reward_fns=[reward_mod7],
                        algo_config=GRPOConfig(num_generations=G, num_iterations=1, beta=0.04, epsilon=0.2))

  rng = np.random.default_rng(100 + rank)

  def batches(n):
    for _ in range(n):
      # prompts are made on the host every step, as a user's data pipeline would deliver them
      ids = rng.integers(1, cfg.vocab_size - 1, size=(per_rank, PL))
      yield {"prompts": [" ".join(map(str, row)) for row in ids]}

  def sync():
    torch.cuda.synchronize()
    if world > 1:
      dist.barrier()
      torch.cuda.synchronize()

  gen_counter = {"n": 0, "rollout_s": 0.0}
  orig_generate = cluster.rollout.generate

  def counting_generate(prompts, rollout_config, **kw):
    t_in = time.perf_counter()
    out = orig_generate(prompts, rollout_config, **kw)       # returns host-side ids: the rollout has finished
    gen_counter["rollout_s"] += time.perf_counter() - t_in
    gen_counter["n"] += int(sum(len(t) for t in out.tokens))
    return out
  cluster.rollout.generate = counting_generate

  data = batches(steps_total)
  # warm-up and timed steps run inside one `train` call (max_steps counts both); a hook marks the boundary
  marks = {}

  class Marks:
    def __init__(self):
      self.step = 0
  state = Marks()
  orig_update = cluster.update_actor
  e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
  sampler = ClockSampler()

  def stepped_iter():
    for i, b in enumerate(data):
      if i == args.warmup:
        sync()
        marks["gen0"] = gen_counter["n"]
        marks["rollout0"] = gen_counter["rollout_s"]
        marks["launch0"] = _lib.launch_calls
        marks["t0"] = time.perf_counter()
        if rank == 0:
          sampler.start()
        e0.record()
      yield b

  learner.train(stepped_iter())
  e1.record()
  sync()
  wall = time.perf_counter() - marks["t0"]
  ms = e0.elapsed_time(e1)
  clocks = sampler.stop(local_rank) if rank == 0 else None
  _lib.check_status()
  gen = gen_counter["n"] - marks["gen0"]
  t = torch.tensor([ms, float(gen), wall], device=dev, dtype=torch.float64)
  if world > 1:
    mx = t.clone()
    dist.all_reduce(mx, op=dist.ReduceOp.MAX)
    sm = t.clone()
    dist.all_reduce(sm, op=dist.ReduceOp.SUM)
    ms, gen, wall = float(mx[0]), float(sm[1]), float(mx[2])
  launches = _lib.launch_calls - marks["launch0"]
  if rank == 0:
    losses = cluster.actor_trainer.metrics_logger.get_metric_history("", "loss", "train")
    out = {
        "metric": "GRPO step tokens/s (rollout + reference log-probs + policy update), generated tokens",
        "value": gen / (ms / 1e3), "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic uniform token ids, random-init weights, reward = share of ids = 0 mod 7",
        "impl": "ours",
        "config": {"model": model_name, "layers": cfg.num_layers, "prompts": P, "generations": G, "prompt_len": PL,
                   "max_new_tokens": NEW,
                   "parallelism": (f"rollout tp{tp} x dp{world // tp} (in-kernel all-reduce exits), trainer fsdp{world}"
                                   if tp > 1 else f"rollout dp{world} on the trainer's replica, trainer fsdp{world}"),
                   "train_micro_prompts": args.grpo_train_micro, "rollout_batch": args.grpo_rollout_batch,
                   "weight_sync": ("every step: re-sharding copy kernel, flat trainer store -> tensor-parallel slice"
                                   if tp > 1 else "none needed: rollout reads the trainer's bf16 replica in place"),
                   "weight_sync_ms": cluster.weight_sync_ms(),
                   "l2": "inputs larger than L2: every decode step streams the 16 GB weights and the KV cache"},
        "generated_tokens_per_step": gen / args.steps,
        "phases_rank0": {"rollout_s_per_step": (gen_counter["rollout_s"] - marks["rollout0"]) / args.steps,
                         "scoring_and_update_s_per_step": (wall - (gen_counter["rollout_s"] - marks["rollout0"]))
                         / args.steps},
        "clocks": clocks,
        "e2e": {"value": gen / wall, "unit": "tokens/s",
                "h2d_bytes_per_step": P * PL * 8 + P * G * (PL + NEW) * 8 * 3,
                "d2h_bytes_per_step": P * G * NEW * 12,
                "note": "the timed region is the public GRPOLearner.train call: prompts arrive as host strings, "
                        "sampled ids and log-probs come back to the host for rewards and advantages every step"},
        "gpu_launches": launches, "train_losses": [float(x) for x in losses],
        "peak_mem_gb": torch.cuda.max_memory_allocated() / 2**30,
    }
    print(json.dumps(out))
  if world > 1:
    dist.barrier()
    dist.destroy_process_group()
