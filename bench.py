"""Headline benchmark: Llama-3.1-8B full-weight SFT (bf16 compute, fp32 master weights + AdamW),
sequence length 4096, global batch 64 sequences, synthetic tokens, random-init weights.

    python bench.py --gpus N --steps K --warmup W          # this framework
    python bench.py --impl reference ...                   # the unmodified reference, if importable

For N > 1 it is launched under torchrun (one rank per GPU, NCCL); ranks shard the model and the
batch (FSDP). Rank 0 prints one JSON line. `value` is total tokens/s over all GPUs, timed on the
device with CUDA events around exactly K optimizer steps (max over ranks); `e2e` repeats the
measurement through `PeftTrainer.train` with inputs copied from pinned host memory every step
and the loss read back to the host.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def parse_args():
  ap = argparse.ArgumentParser()
  ap.add_argument("--gpus", type=int, default=1)
  ap.add_argument("--steps", type=int, default=2)
  ap.add_argument("--warmup", type=int, default=3)
  ap.add_argument("--impl", default="ours", choices=["ours", "reference", "torch_baseline"],
                  help="ours: this framework; reference: the unmodified reference from baseline/_ref; torch_baseline: "
                       "the same step on stock PyTorch (fully_shard over NCCL, cuBLAS, library attention)")
  ap.add_argument("--model", default=None, help="default: llama3p1_8b (sft), qwen3_30b_a3b (moe)")
  ap.add_argument("--seq-len", type=int, default=4096)
  ap.add_argument("--global-batch", type=int, default=0, help="default: 64 (sft), 32 (moe)")
  ap.add_argument("--moe-capacity-factor", type=float, default=2.5,
                  help="expert-parallel receive buffer, in multiples of a rank's own routed rows (overflow is an error)")
  ap.add_argument("--micro-batch", type=int, default=0, help="sequences per micro-step per GPU (0 = auto)")
  ap.add_argument("--layers", type=int, default=0, help="debug only: override the layer count (invalidates the number)")
  ap.add_argument("--remat", default="auto", choices=["auto", "none", "block"])
  ap.add_argument("--no-e2e", action="store_true")
  ap.add_argument("--fsdp-mode", default="resident", choices=["resident", "sharded"],
                  help="sharded: decoder-layer parameters and gradients exist per rank only as 1/N slices, gathered "
                       "layer by layer (tunix_b200/dist/fsdp_sharded.py); resident: whole bf16 replica per rank")
  ap.add_argument("--workload", default="sft", choices=["sft", "grpo", "dpo", "moe"],
                  help="sft: Llama-3.1-8B full-weight SFT (default, the headline); grpo: Qwen3-8B GRPO step; "
                       "dpo: Qwen3-4B DPO with LoRA")
  ap.add_argument("--dpo-pairs", type=int, default=32)
  ap.add_argument("--dpo-prompt-len", type=int, default=512)
  ap.add_argument("--dpo-response-len", type=int, default=512)
  ap.add_argument("--dpo-micro", type=int, default=4, help="pairs per micro-step per GPU")
  ap.add_argument("--grpo-prompts", type=int, default=64)
  ap.add_argument("--grpo-generations", type=int, default=8)
  ap.add_argument("--grpo-prompt-len", type=int, default=256)
  ap.add_argument("--grpo-new-tokens", type=int, default=768)
  ap.add_argument("--grpo-train-micro", type=int, default=1, help="prompts (x generations) per training micro-step")
  ap.add_argument("--grpo-rollout-batch", type=int, default=512, help="sequences decoded together per rank")
  ap.add_argument("--rollout-tp", type=int, default=1,
                  help="grpo: tensor-parallel degree of the rollout engine (rollout data parallelism = GPUs / this); the "
                       "trainer's weights are re-sharded into the rollout layout every step")
  return ap.parse_args()


def reference_arm(args) -> None:
  """Runs the unmodified reference from baseline/_ref through its own API (`baseline/reference_runner.py`).
  Where the reference or the JAX stack under it does not import, or its run fails, rank 0 prints the
  `unavailable` line instead and the process exits 0."""
  from baseline import reference_runner
  rank = int(os.environ.get("RANK", "0"))
  why = reference_runner.probe()
  if why is None and args.workload != "sft":
    why = f"the reference runner covers the SFT workload only, not {args.workload!r}"
  if why is not None:
    if rank == 0:
      print(json.dumps({"impl": "reference", "unavailable": why}))
    return
  gb, micro = args.global_batch or 64, args.micro_batch or 2
  sampler = ClockSampler()
  sampler.start()
  try:
    r = reference_runner.run(n_gpus=args.gpus, steps=args.steps, warmup=args.warmup, global_batch=gb,
                             seq_len=args.seq_len, micro_batch_per_gpu=micro, model_name=args.model or "llama3p1_8b")
  except Exception as e:  # noqa: BLE001 - the arm never takes the bench down
    sampler.stop()
    if rank == 0:
      print(json.dumps({"impl": "reference", "unavailable": f"reference run failed: {type(e).__name__}: {str(e)[:300]}"}))
    return
  clocks = sampler.stop(int(os.environ.get("LOCAL_RANK", "0")))
  if rank == 0:
    print(json.dumps({
        "metric": "SFT tokens/s (Llama-3.1-8B full-weight, bf16 + fp32 master AdamW, seq 4096, global batch 64)",
        "value": r["tokens_per_s"], "unit": "tokens/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": r["ms_per_step"], "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic uniform token ids, random-init N(0,0.02) weights", "impl": "reference",
        "config": {"model": args.model or "llama3p1_8b", "global_batch": gb, "seq_len": args.seq_len,
                   "parallelism": f"fsdp{args.gpus} (reference mesh ({args.gpus},1) over ('fsdp','tp'))",
                   "micro_batch_per_gpu": micro, "grad_accum": r["accum"],
                   "timing": "host clock around PeftTrainer.train with the device drained on both sides; the "
                             "reference exposes no device-side step timer"},
        "clocks": clocks,
        "e2e": {"value": r["tokens_per_s"], "unit": "tokens/s", "h2d_bytes_per_step": r["h2d_bytes_per_step"],
                "d2h_bytes_per_step": 4, "note": "same measurement: inputs come from host memory every micro-step"},
        "gpu_launches": None}))


class ClockSampler:
  """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

  Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
       "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
       "clocks_event_reasons.sw_power_cap")

  def __init__(self):
    self.f = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
    self.p = None

  def start(self):
    try:
      self.p = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "200"],
                                stdout=self.f, stderr=subprocess.DEVNULL)
    except Exception:
      self.p = None

  def stop(self, device_index: int = 0):
    if self.p is None:
      return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
    self.p.terminate()
    try:
      self.p.wait(timeout=5)
    except Exception:
      self.p.kill()
    self.f.flush()
    self.f.seek(0)
    sm, mx, reasons = [], [], set()
    names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
    for line in self.f.read().splitlines():
      parts = [x.strip() for x in line.split(",")]
      if len(parts) < 9:
        continue
      try:
        if int(parts[0]) != device_index:
          continue
        sm.append(float(parts[1]))
        mx.append(float(parts[2]))
      except ValueError:
        continue
      for n, v in zip(names, parts[5:9]):
        if v.lower().startswith("active"):
          reasons.add(n)
    os.unlink(self.f.name)
    return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
            "reasons": sorted(reasons), "samples": len(sm)}


def main():
  args = parse_args()
  if args.impl == "reference":
    reference_arm(args)
    return
  if args.impl == "torch_baseline":
    from baseline import torch_baseline
    torch_baseline.run(args, ClockSampler)
    return
  if args.workload == "dpo":
    from benchmarks import dpo_bench
    dpo_bench.run(args, ClockSampler)
    return
  if args.workload == "grpo":
    from benchmarks import grpo_bench
    grpo_bench.run(args, ClockSampler)
    return

  # micro-batches of 2 sequences need the allocator to grow segments in place: with fixed-size
  # segments the ~150 GiB working set fragments and the step runs out of memory
  os.environ.setdefault("PYTORCH_CUDA_ALLOC_CONF", "expandable_segments:True")
  import torch
  import torch.distributed as dist
  from tunix_b200 import optim
  from tunix_b200.common.configs import TrainingConfig
  from tunix_b200.dist import mesh as mesh_lib
  from tunix_b200.models import flops as flops_lib
  from tunix_b200.models.llama3 import model as llama
  from tunix_b200.models.transformer import RematConfig, Transformer
  from tunix_b200.ops import _lib
  from tunix_b200.sft import hooks as hooks_lib
  from tunix_b200.sft.peft_trainer import PeftTrainer, TrainingInput

  world = int(os.environ.get("WORLD_SIZE", "1"))
  rank = int(os.environ.get("RANK", "0"))
  local_rank = int(os.environ.get("LOCAL_RANK", "0"))
  if world != args.gpus and world > 1:
    raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
  torch.cuda.set_device(local_rank)
  dev = torch.device("cuda", local_rank)
  mesh = None
  if world > 1:
    mesh_lib.init_distributed("nccl")
    mesh = mesh_lib.create_mesh((world,), ("fsdp",))
    mesh_lib.set_current_mesh(mesh)

  moe = args.workload == "moe"
  args.model = args.model or ("qwen3_30b_a3b" if moe else "llama3p1_8b")
  args.global_batch = args.global_batch or (32 if moe else 64)
  if moe:
    from tunix_b200.models.qwen3 import model as qwen3
    cfg = getattr(qwen3.ModelConfig, args.model)()
    full_layers = cfg.num_layers
    if not args.layers and world < 8:
      # the 30B model's optimizer state needs all 8 GPUs; fewer GPUs run proportionally fewer layers (flagged below)
      args.layers = max(1, cfg.num_layers * world // 8)
  else:
    cfg = getattr(llama.ModelConfig, args.model)()
  if args.layers:
    cfg = cfg.replace(num_layers=args.layers)
  S, GB = args.seq_len, args.global_batch
  per_gpu = GB // world
  remat = args.remat
  if remat == "auto":
    remat = "none"      # the fused decoder-layer node stores only what is expensive to rebuild
  micro = args.micro_batch or min(per_gpu, 1 if moe else (2 if remat == "none" else 4))   # MoE keeps routed-row buffers per layer
  ga = per_gpu // micro
  cfg = cfg.replace(dtype=torch.bfloat16, max_position=S,
                    remat_config=RematConfig.BLOCK if remat == "block" else RematConfig.NONE)

  torch.manual_seed(1234)
  model = Transformer(cfg, device=dev).init_weights(seed=0, scale=0.02)
  tx = optim.adamw(learning_rate=1e-5, b1=0.9, b2=0.95, eps=1e-8, weight_decay=0.1)
  tcfg = TrainingConfig(eval_every_n_steps=10**9, gradient_accumulation_steps=ga, max_grad_norm=1.0,
                        pbar_description=None, max_inflight_computations=2 * ga,
                        data_sharding_axis=())   # every rank already holds only its share of the batch
  from tunix_b200.dist import fsdp
  if moe and world > 1:
    from tunix_b200.dist import moe as dist_moe
    dist_moe.shard_experts(model, mesh)      # experts split over the ranks, tokens exchanged over peer memory
    for mod in model.modules():
      if hasattr(mod, "ep_group"):
        mod.ep_capacity_factor = args.moe_capacity_factor
  sharded = args.fsdp_mode == "sharded" and not moe
  model = fsdp.shard_model(model, mesh, mode="sharded" if sharded else "resident")
  trainer = PeftTrainer(model, tx, tcfg)
  trainer.with_grad_sync(fsdp.GradSync(model, mesh))
  trainer.is_managed_externally = True

  # Synthetic data: uniform token ids from a seed, loss on all tokens. This rank's share only.
  g = torch.Generator().manual_seed(1000 + rank)

  def host_batch():
    tok = torch.randint(0, cfg.vocab_size, (micro, S), generator=g, dtype=torch.int32).pin_memory()
    msk = torch.ones((micro, S), dtype=torch.uint8).pin_memory()
    return tok, msk

  def to_input(tok, msk):
    return TrainingInput(input_tokens=tok.to(dev, non_blocking=True).long(), input_mask=msk.to(dev, non_blocking=True))

  n_host = ga * 2
  host = [host_batch() for _ in range(n_host)]
  resident = [to_input(*hb) for hb in host]

  def dev_dataset(n_steps):
    for i in range(n_steps * ga):
      yield resident[i % n_host]

  def host_dataset(n_steps):
    for i in range(n_steps * ga):
      tok, msk = host[i % n_host]
      yield TrainingInput(input_tokens=tok, input_mask=msk)   # copied H2D inside the trainer, every step

  def sync():
    torch.cuda.synchronize()
    if world > 1:
      dist.barrier()
      torch.cuda.synchronize()

  # ---- device-timed region --------------------------------------------------------------
  trainer.train(dev_dataset(args.warmup))
  sync()
  sampler = ClockSampler()
  if rank == 0:
    sampler.start()
  launches0 = _lib.launch_calls
  e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
  e0.record()
  trainer.train(dev_dataset(args.steps))
  e1.record()
  sync()
  ms = e0.elapsed_time(e1)
  launches = _lib.launch_calls - launches0
  clocks = sampler.stop(local_rank) if rank == 0 else None
  need = None
  if moe and world > 1:
    from tunix_b200.dist import moe as dist_moe
    need = dist_moe.peak_capacity_need()
    if need is not None and need > args.moe_capacity_factor:
      raise SystemExit(f"rank {rank}: expert-parallel receive buffer too small: this routing needs a capacity factor of "
                       f"{need:.2f} (--moe-capacity-factor {args.moe_capacity_factor}); rows beyond it were dropped, "
                       "so the run is invalid")
  _lib.check_status()
  t = torch.tensor([ms], device=dev)
  if world > 1:
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
  ms_total = float(t.item())
  tokens_per_step = GB * S
  value = tokens_per_step * args.steps / (ms_total / 1e3)

  # ---- end to end through the public API ---------------------------------------------------
  e2e = None
  if not args.no_e2e:
    class ReadLoss(hooks_lib.TrainingHooks):
      """Reads the step's loss back to the host (the trainer hands over a host float)."""
      def __init__(self):
        self.losses = []
      def on_train_step_end(self, ctx, step, loss):
        self.losses.append(float(loss))
    rl = ReadLoss()
    trainer.with_training_hooks(rl)
    trainer.train(host_dataset(1))       # one warm step through the host path
    sync()
    t0 = time.perf_counter()
    trainer.train(host_dataset(args.steps))
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    tt = torch.tensor([dt], device=dev)
    if world > 1:
      dist.all_reduce(tt, op=dist.ReduceOp.MAX)
    dt = float(tt.item())
    h2d = GB * S * (4 + 1)      # int32 tokens + uint8 mask, whole job per optimizer step
    d2h = 8 * world            # fp32 loss + fp32 grad-norm per rank per optimizer step
    e2e = {"value": tokens_per_step * args.steps / dt, "unit": "tokens/s", "h2d_bytes_per_step": h2d,
           "d2h_bytes_per_step": d2h, "losses": rl.losses[-args.steps:]}

  if rank == 0:
    fl = flops_lib.train_flops_per_token(cfg, S) * tokens_per_step
    metric = "SFT tokens/s (Llama-3.1-8B full-weight, bf16 + fp32 master AdamW, seq 4096, global batch 64)"
    if (args.model, S, GB, cfg.num_layers) != ("llama3p1_8b", 4096, 64, 32) and not moe:
      metric = (f"SFT tokens/s ({args.model}, {cfg.num_layers} layers, full-weight, bf16 + fp32 master AdamW, seq {S}, "
                f"global batch {GB}) - not the headline configuration")
    if moe:
      metric = (f"SFT tokens/s (Qwen3-30B-A3B MoE full-weight, expert parallel over {world} GPU(s), bf16 + fp32 master "
                f"AdamW, seq {S}, global batch {GB})")
    out = {
        "metric": metric,
        "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_total / args.steps, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic uniform token ids, random-init N(0,0.02) weights",
        "impl": "ours",
        "config": {"model": args.model, "layers": cfg.num_layers, "global_batch": GB, "seq_len": S,
                   "parallelism": f"ep{world}+fsdp{world}" if moe else f"fsdp{world}" + ("-sharded-params" if sharded else ""),
                   "fsdp_mode": "sharded" if sharded else "resident",
                   "sharding": ("decoder-layer parameters (bf16), gradient accumulators (fp32), fp32 master and Adam moments "
                                "all sharded over the ranks; a layer is gathered for its forward and again for its backward "
                                "(NCCL all-gather prefetched on a side stream), its gradients reduce-scattered as soon as its "
                                "backward has run; embedding / final norm / head stay whole on every rank" if sharded else
                                "fp32 master / Adam moments and the reduced gradient are sharded over the ranks (interleaved by "
                                "bucket); every rank keeps a resident bf16 parameter replica and its own fp32 gradient "
                                "accumulator" if world > 1 else "single GPU"),
                   "micro_batch_per_gpu": micro, "grad_accum": ga, "remat": remat,
                   "l2": "inputs larger than L2: each step streams >100 GB of weights, gradients and optimizer state",
                   "optimizer": "AdamW fp32 master/m/v, global-norm clip 1.0"},
        **({"moe": {"full_model_layers": full_layers, "layers_run": cfg.num_layers,
                    "reduced": cfg.num_layers != full_layers, "experts": cfg.num_experts,
                    "top_k": cfg.num_experts_per_tok, "capacity_factor": args.moe_capacity_factor,
                    "capacity_needed_rank0": need}} if moe else {}),
        "model_tflops_per_gpu": fl / (ms_total / args.steps / 1e3) / 1e12 / world,
        "clocks": clocks, "e2e": e2e, "gpu_launches": launches,
        "train_losses": [float(x) for x in trainer.metrics_logger.get_metric_history("", "loss", "train")[:args.warmup + args.steps]],
        "peak_mem_gb": torch.cuda.max_memory_allocated() / 2**30,
        # the caching allocator does not see symmetric (peer-mapped) buffers: flat parameters, gradients, exchange buffers
        "device_mem_in_use_gb": (lambda fr_to: (fr_to[1] - fr_to[0]) / 2**30)(torch.cuda.mem_get_info()),
    }
    print(json.dumps(out))
  if world > 1:
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
  main()
